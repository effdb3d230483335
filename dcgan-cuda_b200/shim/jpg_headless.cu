// Headless stand-in for the reference's src/datasets/jpg.cu (libjpeg is not part of this
// build): same img:: interface (src/datasets/jpg.hh).  Saving writes a binary PPM (P6) next to the
// requested path ("<path>.ppm"); loading is refused - the training binaries then need their
// inputs from a tensor archive or a synthetic source instead of a directory of JPEG files.
#include "datasets/jpg.hh"

#include <cstdio>
#include <stdexcept>

namespace img
{

    std::uint8_t* jpg_load(const std::string& path, std::size_t*, std::size_t*, std::size_t*)
    {
        throw std::runtime_error("jpg_load(" + path + "): this build has no JPEG decoder");
    }

    void jpg_save(const std::string& path, std::uint8_t* data, std::size_t width, std::size_t height, int)
    {
        const std::string out = path + ".ppm";
        std::FILE* f = std::fopen(out.c_str(), "wb");
        if (!f) throw std::runtime_error("jpg_save: cannot write " + out);
        std::fprintf(f, "P6\n%zu %zu\n255\n", width, height);
        const std::size_t n = width * height * 3;
        const bool ok = std::fwrite(data, 1, n, f) == n;
        if (std::fclose(f) != 0 || !ok) throw std::runtime_error("jpg_save: write failed: " + out);
    }

}

// Converts a tensor archive: reads IN (an .npz written by numpy.savez, or the raw archive of
// tocha/tensor.hh) and writes OUT as a raw archive.  Usage: archive_tool IN OUT
#include <cstdio>
#include <exception>

#include <tocha/tensor.hh>

int main(int argc, char** argv)
{
    if (argc != 3) {
        std::fprintf(stderr, "usage: %s IN OUT\n", argv[0]);
        return 2;
    }
    try {
        auto ts = tocha::Tensors::load(argv[1]);
        ts.save(argv[2]);
        std::printf("%zu tensors\n", ts.arr().size());
    } catch (const std::exception& e) {
        std::fprintf(stderr, "%s\n", e.what());
        return 1;
    }
    return 0;
}

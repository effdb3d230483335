// Stand-in for the reference's un-vendored tensor-archive dependency (ext/tocha, an empty git
// submodule): just the surface the reference's sources use - tocha::Tensor::f32(d0[,d1[,d2[,d3]]][,ptr]),
// Tensor::data, Tensor::dims, tocha::Tensors::{add, arr, save, load} (src/ops/graph.cu:326-361,
// tests/test_reshape.cu:38-49, tests/test_dcgan_discriminator.cu:26-28).
//
// File formats:
//  * save() writes a raw little-endian archive: "DCGT", u32 version 1, u32 tensor count, then per
//    tensor u32 rank, rank x u32 extents, the fp32 values.  load() reads it back.  (The byte layout
//    of tocha's own .tbin files is not known here; this archive only promises to read what it wrote.)
//  * load() also reads an .npz written by numpy.savez (a zip of STORED, uncompressed .npy members,
//    fp32 or fp64, C order) - what the reference's Python reference scripts hand to its test programs
//    (tests/pyts/tensors_saver.py).  Members are taken in name order, as numpy wrote them.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace tocha
{

    struct Tensor
    {
        std::vector<int> dims;
        std::uint8_t* data = nullptr;       // fp32 values, row-major
        std::size_t total_len = 0;          // number of values
        std::shared_ptr<std::vector<float>> store;   // owner of `data`

        static Tensor make(const std::vector<int>& d, const void* src)
        {
            Tensor t;
            t.dims = d;
            t.total_len = 1;
            for (int e : d) t.total_len *= (std::size_t)e;
            t.store = std::make_shared<std::vector<float>>(t.total_len ? t.total_len : 1, 0.f);
            t.data = reinterpret_cast<std::uint8_t*>(t.store->data());
            if (src) std::memcpy(t.data, src, t.total_len * sizeof(float));
            return t;
        }

        static Tensor f32(std::size_t d0, const void* p = nullptr) { return make({(int)d0}, p); }
        static Tensor f32(std::size_t d0, std::size_t d1, const void* p = nullptr) { return make({(int)d0, (int)d1}, p); }
        static Tensor f32(std::size_t d0, std::size_t d1, std::size_t d2, const void* p = nullptr)
        {
            return make({(int)d0, (int)d1, (int)d2}, p);
        }
        static Tensor f32(std::size_t d0, std::size_t d1, std::size_t d2, std::size_t d3, const void* p = nullptr)
        {
            return make({(int)d0, (int)d1, (int)d2, (int)d3}, p);
        }
    };

    class Tensors
    {
    public:
        void add(const Tensor& t) { arr_.push_back(t); }
        std::vector<Tensor>& arr() { return arr_; }
        const std::vector<Tensor>& arr() const { return arr_; }

        void save(const std::string& path) const
        {
            std::FILE* f = std::fopen(path.c_str(), "wb");
            if (!f) throw std::runtime_error("tocha stub: cannot write " + path);
            const std::uint32_t head[2] = {1u, (std::uint32_t)arr_.size()};
            bool ok = std::fwrite("DCGT", 1, 4, f) == 4 && std::fwrite(head, 4, 2, f) == 2;
            for (const Tensor& t : arr_) {
                const std::uint32_t rank = (std::uint32_t)t.dims.size();
                ok = ok && std::fwrite(&rank, 4, 1, f) == 1;
                std::size_t n = 1;
                for (int e : t.dims) {
                    const std::uint32_t u = (std::uint32_t)e;
                    ok = ok && std::fwrite(&u, 4, 1, f) == 1;
                    n *= (std::size_t)e;
                }
                ok = ok && (n == 0 || std::fwrite(t.data, sizeof(float), n, f) == n);
            }
            if (std::fclose(f) != 0 || !ok) throw std::runtime_error("tocha stub: write failed: " + path);
        }

        static Tensors load(const std::string& path)
        {
            std::vector<std::uint8_t> buf = slurp(path);
            if (buf.size() >= 12 && std::memcmp(buf.data(), "DCGT", 4) == 0) return load_raw(buf, path);
            if (buf.size() >= 4 && buf[0] == 'P' && buf[1] == 'K') return load_npz(buf, path);
            throw std::runtime_error("tocha stub: " + path + " is neither a raw archive nor an .npz");
        }

    private:
        std::vector<Tensor> arr_;

        static std::vector<std::uint8_t> slurp(const std::string& path)
        {
            std::FILE* f = std::fopen(path.c_str(), "rb");
            if (!f) throw std::runtime_error("tocha stub: cannot read " + path);
            std::vector<std::uint8_t> buf;
            std::uint8_t chunk[1 << 16];
            std::size_t got;
            while ((got = std::fread(chunk, 1, sizeof(chunk), f)) > 0) buf.insert(buf.end(), chunk, chunk + got);
            std::fclose(f);
            return buf;
        }

        static std::uint32_t u32(const std::vector<std::uint8_t>& b, std::size_t off)
        {
            if (off + 4 > b.size()) throw std::runtime_error("tocha stub: truncated archive");
            std::uint32_t v;
            std::memcpy(&v, b.data() + off, 4);
            return v;
        }
        static std::uint16_t u16(const std::vector<std::uint8_t>& b, std::size_t off)
        {
            if (off + 2 > b.size()) throw std::runtime_error("tocha stub: truncated archive");
            std::uint16_t v;
            std::memcpy(&v, b.data() + off, 2);
            return v;
        }

        static Tensors load_raw(const std::vector<std::uint8_t>& b, const std::string& path)
        {
            if (u32(b, 4) != 1u) throw std::runtime_error("tocha stub: unknown archive version in " + path);
            const std::uint32_t count = u32(b, 8);
            std::size_t off = 12;
            Tensors out;
            for (std::uint32_t i = 0; i < count; ++i) {
                const std::uint32_t rank = u32(b, off);
                off += 4;
                std::vector<int> dims;
                std::size_t n = 1;
                for (std::uint32_t r = 0; r < rank; ++r) {
                    dims.push_back((int)u32(b, off));
                    n *= (std::size_t)dims.back();
                    off += 4;
                }
                if (off + n * 4 > b.size()) throw std::runtime_error("tocha stub: truncated archive " + path);
                out.add(Tensor::make(dims, b.data() + off));
                off += n * 4;
            }
            return out;
        }

        // numpy.savez: local file headers (signature 0x04034b50) with method 0 (stored); sizes may sit
        // in a zip64 extra field when numpy streams the member.  The central directory is used for
        // the member list because it always carries the final sizes.
        static Tensors load_npz(const std::vector<std::uint8_t>& b, const std::string& path)
        {
            std::size_t eocd = std::string::npos;
            for (std::size_t i = b.size() >= 22 ? b.size() - 22 : 0;; --i) {
                if (u32(b, i) == 0x06054b50u) { eocd = i; break; }
                if (i == 0) break;
            }
            if (eocd == std::string::npos) throw std::runtime_error("tocha stub: no zip directory in " + path);
            std::size_t n_entries = u16(b, eocd + 10), cd_off = u32(b, eocd + 16);
            if (cd_off == 0xFFFFFFFFu || n_entries == 0xFFFFu) {   // zip64 end record
                for (std::size_t i = eocd; i-- > 0;) {
                    if (u32(b, i) == 0x06064b50u) {
                        std::uint64_t v;
                        std::memcpy(&v, b.data() + i + 32, 8); n_entries = (std::size_t)v;
                        std::memcpy(&v, b.data() + i + 48, 8); cd_off = (std::size_t)v;
                        break;
                    }
                }
            }
            struct Member { std::string name; std::size_t local, size; };
            std::vector<Member> members;
            std::size_t off = cd_off;
            for (std::size_t e = 0; e < n_entries; ++e) {
                if (u32(b, off) != 0x02014b50u) throw std::runtime_error("tocha stub: bad zip directory in " + path);
                if (u16(b, off + 10) != 0) throw std::runtime_error("tocha stub: compressed .npz member in " + path + " (use numpy.savez, not savez_compressed)");
                std::uint64_t size = u32(b, off + 24), local = u32(b, off + 42);
                const std::size_t nlen = u16(b, off + 28), xlen = u16(b, off + 30), clen = u16(b, off + 32);
                std::string name(reinterpret_cast<const char*>(b.data() + off + 46), nlen);
                std::size_t x = off + 46 + nlen;
                const std::size_t xend = x + xlen;
                while (x + 4 <= xend) {   // zip64 extra: uncompressed, compressed, local offset - each only if the 32-bit field is all ones
                    const std::uint16_t id = u16(b, x), len = u16(b, x + 2);
                    if (id == 0x0001) {
                        std::size_t q = x + 4;
                        if (u32(b, off + 24) == 0xFFFFFFFFu) { std::memcpy(&size, b.data() + q, 8); q += 8; }
                        if (u32(b, off + 20) == 0xFFFFFFFFu) q += 8;
                        if (u32(b, off + 42) == 0xFFFFFFFFu) { std::memcpy(&local, b.data() + q, 8); }
                    }
                    x += 4 + len;
                }
                members.push_back({name, (std::size_t)local, (std::size_t)size});
                off += 46 + nlen + xlen + clen;
            }
            std::sort(members.begin(), members.end(), [](const Member& a, const Member& c) { return a.name < c.name; });
            Tensors out;
            for (const Member& m : members) {
                if (u32(b, m.local) != 0x04034b50u) throw std::runtime_error("tocha stub: bad zip member in " + path);
                const std::size_t data = m.local + 30 + u16(b, m.local + 26) + u16(b, m.local + 28);
                if (data + m.size > b.size()) throw std::runtime_error("tocha stub: truncated .npz " + path);
                out.add(parse_npy(b.data() + data, m.size, path + ":" + m.name));
            }
            return out;
        }

        static Tensor parse_npy(const std::uint8_t* p, std::size_t n, const std::string& what)
        {
            if (n < 10 || std::memcmp(p, "\x93NUMPY", 6) != 0) throw std::runtime_error("tocha stub: not an .npy member: " + what);
            std::size_t hlen, hoff;
            if (p[6] == 1) { hlen = p[8] | (p[9] << 8); hoff = 10; }
            else { std::uint32_t h; std::memcpy(&h, p + 8, 4); hlen = h; hoff = 12; }
            const std::string head(reinterpret_cast<const char*>(p + hoff), hlen);
            const bool f4 = head.find("'<f4'") != std::string::npos, f8 = head.find("'<f8'") != std::string::npos;
            if (!f4 && !f8) throw std::runtime_error("tocha stub: .npy member is not little-endian fp32/fp64: " + what);
            if (head.find("'fortran_order': False") == std::string::npos)
                throw std::runtime_error("tocha stub: Fortran-ordered .npy member: " + what);
            const std::size_t s0 = head.find("'shape': ("), s1 = head.find(')', s0);
            if (s0 == std::string::npos || s1 == std::string::npos) throw std::runtime_error("tocha stub: no shape in " + what);
            std::vector<int> dims;
            std::size_t count = 1;
            const std::string shape = head.substr(s0 + 10, s1 - s0 - 10);
            for (std::size_t i = 0; i < shape.size();) {
                if (shape[i] < '0' || shape[i] > '9') { ++i; continue; }
                long v = 0;
                while (i < shape.size() && shape[i] >= '0' && shape[i] <= '9') v = v * 10 + (shape[i++] - '0');
                dims.push_back((int)v);
                count *= (std::size_t)v;
            }
            if (dims.empty()) dims.push_back(1);   // 0-d array: one value
            const std::uint8_t* body = p + hoff + hlen;
            if (hoff + hlen + count * (f4 ? 4 : 8) > n) throw std::runtime_error("tocha stub: truncated .npy member: " + what);
            Tensor t = Tensor::make(dims, f4 ? body : nullptr);
            if (f8) {
                float* dst = reinterpret_cast<float*>(t.data);
                for (std::size_t i = 0; i < count; ++i) {
                    double v;
                    std::memcpy(&v, body + 8 * i, 8);
                    dst[i] = (float)v;
                }
            }
            return t;
        }
    };

}

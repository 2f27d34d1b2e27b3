// mmap reader for safetensors files with byte-range shard slicing and fp8 block dequant.
//
// A safetensors file is an 8-byte little-endian header length, a JSON header
// {name: {dtype, shape, data_offsets:[begin,end]}} and the raw tensor bytes.  The reader maps
// the file once; tensors are handed out as zero-copy views or copied by row/column byte
// ranges straight into the caller's (pinned) buffer, so a tensor-parallel shard never
// materialises the full tensor (reference crates/ferrite-model/src/safetensors.rs:63-115,
// direct.rs:154-497, crates/ferrite-models/src/dsv41/load.rs:394-1228).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

namespace fbrt {

inline float e4m3_to_f32(uint8_t v) {
    const int s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
    float f;
    if (e == 0) f = std::ldexp((float)m, -9);                 // subnormal: m/8 * 2^-6
    else if (e == 15 && m == 7) f = NAN;                      // the only NaN of e4m3fn
    else f = std::ldexp(1.f + m / 8.f, e - 7);
    return s ? -f : f;
}

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path) : path_(path) {
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) throw std::runtime_error("cannot open " + path);
        struct stat st;
        if (fstat(fd_, &st) != 0 || st.st_size < 8) { ::close(fd_); throw std::runtime_error("bad safetensors file " + path); }
        size_ = (size_t)st.st_size;
        base_ = (const uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (base_ == MAP_FAILED) { ::close(fd_); throw std::runtime_error("mmap failed for " + path); }
        uint64_t n = 0;
        std::memcpy(&n, base_, 8);
        if (n == 0 || 8 + n > size_) { cleanup(); throw std::runtime_error("corrupt safetensors header in " + path); }
        header_.assign((const char*)base_ + 8, (size_t)n);
        data_ = 8 + (size_t)n;
    }
    ~SafetensorsFile() { cleanup(); }
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;

    const std::string& header() const { return header_; }
    size_t data_offset() const { return data_; }
    size_t data_size() const { return size_ - data_; }
    const uint8_t* data() const { return base_ + data_; }

    // Copy rows [r0, r1) and byte columns [c0, c1) of a row-major tensor that starts at data
    // offset `begin` with `row_bytes` bytes per row.
    void copy_rows(size_t begin, size_t row_bytes, size_t r0, size_t r1, size_t c0, size_t c1, uint8_t* dst) const {
        if (c1 > row_bytes || c0 > c1 || begin + r1 * row_bytes > data_size()) throw std::out_of_range("copy_rows range");
        const size_t w = c1 - c0;
        for (size_t r = r0; r < r1; ++r) std::memcpy(dst + (r - r0) * w, data() + begin + r * row_bytes + c0, w);
    }

    // e4m3 [rows, cols] at `begin` with f32 scales [ceil(rows/blk), ceil(cols/blk)] at
    // `scale_begin` -> f32 rows [r0, r1) into dst.
    void dequant_e4m3_block(size_t begin, size_t scale_begin, size_t rows, size_t cols, size_t blk, size_t r0,
                            size_t r1, float* dst) const {
        if (blk == 0) throw std::out_of_range("dequant block size");
        const size_t kb = (cols + blk - 1) / blk, rb = (rows + blk - 1) / blk;
        if (begin + rows * cols > data_size() || r1 > rows || r0 > r1) throw std::out_of_range("dequant range");
        if (scale_begin + rb * kb * sizeof(float) > data_size()) throw std::out_of_range("dequant scale range");
        // tensor data in a safetensors file is only byte-aligned: read the scales through memcpy
        const uint8_t* sc = data() + scale_begin;
        for (size_t r = r0; r < r1; ++r) {
            const uint8_t* src = data() + begin + r * cols;
            for (size_t cb = 0; cb < kb; ++cb) {
                float scale;
                std::memcpy(&scale, sc + ((r / blk) * kb + cb) * sizeof(float), sizeof(float));
                const size_t c1 = std::min(cols, (cb + 1) * blk);
                for (size_t c = cb * blk; c < c1; ++c) dst[(r - r0) * cols + c] = e4m3_to_f32(src[c]) * scale;
            }
        }
    }

private:
    void cleanup() {
        if (base_ && base_ != MAP_FAILED) munmap((void*)base_, size_);
        if (fd_ >= 0) ::close(fd_);
        base_ = nullptr; fd_ = -1;
    }
    std::string path_, header_;
    int fd_ = -1;
    size_t size_ = 0, data_ = 0;
    const uint8_t* base_ = nullptr;
};

}  // namespace fbrt

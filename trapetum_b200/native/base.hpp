// Shared pieces of the native host: dtypes, matrices as (pointer, shape, stride), device memory, CUDA status.
#pragma once
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstring>

#include "json.hpp"

namespace tb {

enum DType { F32 = 0, BF16 = 1, I32 = 2 };        // 0 and 1 are the codes the kernels take

inline size_t dtype_size(DType d) { return d == BF16 ? 2 : 4; }
inline const char* dtype_name(DType d) { return d == F32 ? "float32" : d == BF16 ? "bfloat16" : "int32"; }

inline void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw Error(fmt("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e)));
}

constexpr int PAGE_ROWS = 64;                     // rows of one cache page (compiled into the attention kernels)

// A matrix [rows, cols] with contiguous rows `ld` elements apart.
struct Mat {
    void* p = nullptr;
    DType dt = F32;
    int64_t rows = 0, cols = 0, ld = 0;
    Mat() {}
    Mat(void* p_, DType d, int64_t r, int64_t c, int64_t ld_ = -1) : p(p_), dt(d), rows(r), cols(c), ld(ld_ < 0 ? c : ld_) {}
    bool contiguous() const { return ld == cols; }
    size_t bytes() const { return (size_t)rows * ld * dtype_size(dt); }
    char* at(int64_t r, int64_t c = 0) const { return (char*)p + ((size_t)r * ld + c) * dtype_size(dt); }
    Mat cols_slice(int64_t c0, int64_t n) const { return Mat(at(0, c0), dt, rows, n, ld); }
    Mat rows_slice(int64_t r0, int64_t n) const { return Mat(at(r0, 0), dt, n, cols, ld); }
    explicit operator bool() const { return p != nullptr; }
};

// 32-bit partial sums [splits, rows, cols] whose sum over the first axis, taken in order, is a product.
struct Partials {
    float* p = nullptr;
    int splits = 1;
    int64_t split_stride = 0, rows = 0, cols = 0;
    Mat first() const { return Mat(p, F32, rows, cols); }
};

// Device memory owned by an object.
struct DeviceBuffer {
    void* p = nullptr;
    size_t bytes = 0;
    DeviceBuffer() {}
    explicit DeviceBuffer(size_t n) { alloc(n); }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : p(o.p), bytes(o.bytes) { o.p = nullptr; o.bytes = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) { release(); p = o.p; bytes = o.bytes; o.p = nullptr; o.bytes = 0; }
        return *this;
    }
    ~DeviceBuffer() { release(); }
    void alloc(size_t n) {
        release();
        if (n == 0) return;
        cudaError_t e = cudaMalloc(&p, n);
        if (e != cudaSuccess) {
            p = nullptr;
            size_t fr = 0, tot = 0;
            cudaMemGetInfo(&fr, &tot);
            cudaGetLastError();
            throw Error(fmt("out of device memory: %.2f GB asked, %.2f of %.2f GB free", n / 1e9, fr / 1e9, tot / 1e9));
        }
        bytes = n;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
};

// Scratch memory of a step: three regions of one allocation.  STEP lives for the whole step; the two LAYER
// regions are used by alternate layers, each reset when its layer begins, so that what a layer leaves for the
// next one (a branch output that is added together with the next norm) stays valid while the next layer runs.
// A step of a new size first runs "dry": the same code path with every kernel launch left out, which only
// counts what it would allocate; the arena then grows to those peaks before the step runs for real.
class Arena {
public:
    enum Region { STEP = 0, LAYER_A = 1, LAYER_B = 2 };
    void reserve(size_t step_bytes, size_t layer_bytes) {
        step_bytes = (step_bytes + 255) & ~(size_t)255;         // every region starts on a 256-byte boundary
        layer_bytes = (layer_bytes + 255) & ~(size_t)255;
        cap_[0] = step_bytes; cap_[1] = cap_[2] = layer_bytes;
        buf_.alloc(step_bytes + 2 * layer_bytes);
        base_[0] = 0; base_[1] = step_bytes; base_[2] = step_bytes + layer_bytes;
        begin_step();
    }
    void begin_step() { used_[0] = used_[1] = used_[2] = 0; peak_[0] = peak_[1] = peak_[2] = 0; cur_ = STEP; }
    void reset(Region r) { used_[r] = 0; }
    void use(Region r) { cur_ = r; }
    Region current() const { return cur_; }
    bool dry = false;
    void* alloc(size_t bytes) { return alloc(bytes, cur_); }
    void* alloc(size_t bytes, Region r) {
        const size_t n = (bytes + 255) & ~(size_t)255;
        used_[r] += n;
        if (used_[r] > peak_[r]) peak_[r] = used_[r];
        if (used_[r] > cap_[r] && !dry)
            throw Error(fmt("step arena: region %d needs %zu bytes, holds %zu (the dry pass should have sized it)",
                            (int)r, used_[r], cap_[r]));
        return (char*)buf_.p + base_[r] + used_[r] - n;          // in a dry pass possibly past the end: never touched
    }
    Mat mat(DType dt, int64_t rows, int64_t cols) { return Mat(alloc((size_t)rows * cols * dtype_size(dt)), dt, rows, cols); }
    Mat mat(DType dt, int64_t rows, int64_t cols, Region r) {
        return Mat(alloc((size_t)rows * cols * dtype_size(dt), r), dt, rows, cols);
    }
    bool fits_peaks() const { return peak_[0] <= cap_[0] && peak_[1] <= cap_[1] && peak_[2] <= cap_[2]; }
    void grow_to_peaks() {
        const size_t layer = std::max(std::max(peak_[1], peak_[2]), cap_[1]);
        const size_t step = std::max(peak_[0], cap_[0]);
        reserve(step + (step >> 4) + 4096, layer + (layer >> 4) + 4096);
    }
    size_t capacity() const { return buf_.bytes; }

private:
    DeviceBuffer buf_;
    size_t cap_[3] = {0, 0, 0}, base_[3] = {0, 0, 0}, used_[3] = {0, 0, 0}, peak_[3] = {0, 0, 0};
    Region cur_ = STEP;
};

}  // namespace tb

// RMSNorm and its fusion with the residual sum.
//
//   y = x * rsqrt(mean(x^2) + eps) * (offset + w)       offset = 1 for the (1+w) form
//
// The reference runs `out = x*rsqrt(mean x^2 + eps)*w` in one 256-thread block
// per call with the +1 pre-added to w at export (runtime/cuda/codebook_gemv.cu:192-202,
// model/export_gemma.py:25-26) and adds the residual in a separate kernel
// (codebook_gemv.cu:539-542).  Here one CTA owns one row; the sum of squares,
// the rsqrt, the scale and the residual sum are all 32-bit, and the fused form
// does `h += norm_a(a); x = norm_b(h)` in one pass over the row:
//
//   tb_rmsnorm      out = norm(x)
//   tb_add_rmsnorm  h (32-bit, in place) += norm_a(a);  then, if asked, out = norm_b(h);
//                   a may be given as split-K partial sums, added here in split order
//
// Any row width works (loops are strided by the block size).
#include "common.cuh"

TB_EXPORT_ERROR()

template <typename TX, typename TW, typename TO>
__global__ void rmsnorm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               int width, float eps, float offset) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { float v = to_f<TX>(x[base + i]); ss += v * v; }
    ss = block_sum(ss, red);
    const float r = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        out[base + i] = from_f<TO>(to_f<TX>(x[base + i]) * r * (offset + to_f<TW>(w[i])));
}

// h += norm_a(a); optionally out = norm_b(h).  `a` may come as n_splits partial sums (32-bit, the
// split-K output of a matrix product, [n_splits][rows][width]); they are added in split order here,
// which saves the separate reduction pass.  The row of `a` is kept in shared memory between the two
// passes over it when it fits (row_cache != 0); a thread re-reads only elements that it wrote itself.
template <typename TA, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TA* __restrict__ a, int n_splits, long long split_stride,
                                   const TW* __restrict__ wa, float eps_a, float off_a,
                                   const TW* __restrict__ wb, float eps_b, float off_b,
                                   TO* __restrict__ out, int width, int row_cache) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row[];
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = to_f<TA>(a[base + i]);
        for (int s = 1; s < n_splits; s++) v += to_f<TA>(a[(size_t)s * split_stride + base + i]);
        if (row_cache) row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float ra = rsqrtf(ss / (float)width + eps_a);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float av;
        if (row_cache) av = row[i];
        else {
            av = to_f<TA>(a[base + i]);
            for (int s = 1; s < n_splits; s++) av += to_f<TA>(a[(size_t)s * split_stride + base + i]);
        }
        const float v = h[base + i] + av * ra * (off_a + to_f<TW>(wa[i]));
        h[base + i] = v;
        if (row_cache) row[i] = v;
        s2 += v * v;
    }
    if (out == nullptr) return;
    s2 = block_sum(s2, red);
    const float rb = rsqrtf(s2 / (float)width + eps_b);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        out[base + i] = from_f<TO>((row_cache ? row[i] : h[base + i]) * rb * (off_b + to_f<TW>(wb[i])));
}

static int norm_threads(int width) {
    int t = 64;
    while (t < 1024 && t * 4 < width) t <<= 1;
    return t;
}

#define DISPATCH3(cx, cw, co, ...)                                                         \
    do {                                                                                   \
        const int key_ = ((cx) << 2) | ((cw) << 1) | (co);                                 \
        switch (key_) {                                                                    \
        case 0: { typedef float TX; typedef float TW; typedef float TO; __VA_ARGS__; } break;   \
        case 1: { typedef float TX; typedef float TW; typedef bf16 TO; __VA_ARGS__; } break;    \
        case 2: { typedef float TX; typedef bf16 TW; typedef float TO; __VA_ARGS__; } break;    \
        case 3: { typedef float TX; typedef bf16 TW; typedef bf16 TO; __VA_ARGS__; } break;     \
        case 4: { typedef bf16 TX; typedef float TW; typedef float TO; __VA_ARGS__; } break;    \
        case 5: { typedef bf16 TX; typedef float TW; typedef bf16 TO; __VA_ARGS__; } break;     \
        case 6: { typedef bf16 TX; typedef bf16 TW; typedef float TO; __VA_ARGS__; } break;     \
        case 7: { typedef bf16 TX; typedef bf16 TW; typedef bf16 TO; __VA_ARGS__; } break;      \
        default: return tb_refuse("norm: unknown dtype codes %d %d %d", (cx), (cw), (co));  \
        }                                                                                  \
    } while (0)

static bool code_ok(int c) { return c == TB_F32 || c == TB_BF16; }

extern "C" int tb_rmsnorm(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                          int rows, int width, float eps, float offset, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return tb_refuse("rmsnorm: width=%d", width);
    if (!code_ok(x_dtype) || !code_ok(w_dtype) || !code_ok(out_dtype))
        return tb_refuse("rmsnorm: unknown dtype codes %d %d %d", x_dtype, w_dtype, out_dtype);
    DISPATCH3(x_dtype, w_dtype, out_dtype,
        tb_launch(rmsnorm_kernel<TX, TW, TO>, dim3(rows), dim3(norm_threads(width)), 0, stream, 
            (const TX*)x, (const TW*)w, (TO*)out, width, eps, offset));
    return tb_launch_status();
}

extern "C" int tb_add_rmsnorm(float* h, const void* a, int a_dtype, int n_splits, long long split_stride,
                              const void* wa, float eps_a, float off_a,
                              const void* wb, float eps_b, float off_b, int w_dtype,
                              void* out, int out_dtype, int rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return tb_refuse("add_rmsnorm: width=%d", width);
    if (!code_ok(a_dtype) || !code_ok(w_dtype) || !code_ok(out_dtype))
        return tb_refuse("add_rmsnorm: unknown dtype codes %d %d %d", a_dtype, w_dtype, out_dtype);
    if (out != nullptr && wb == nullptr) return tb_refuse("add_rmsnorm: an output needs the second norm's weight");
    if (n_splits < 1) return tb_refuse("add_rmsnorm: n_splits=%d", n_splits);
    const int row_cache = (size_t)width * sizeof(float) <= 40 * 1024;
    const size_t smem = row_cache ? (size_t)width * sizeof(float) : 0;
    DISPATCH3(a_dtype, w_dtype, out_dtype,
        tb_launch(add_rmsnorm_kernel<TX, TW, TO>, dim3(rows), dim3(norm_threads(width)), smem, stream,
            h, (const TX*)a, n_splits, split_stride, (const TW*)wa, eps_a, off_a, (const TW*)wb, eps_b, off_b,
            (TO*)out, width, row_cache));
    return tb_launch_status();
}

// h += a, both 32-bit or a in bfloat16: the plain residual sum for arrangements
// that have no norm on the branch output.
template <typename TA>
__global__ void add_kernel(float* __restrict__ h, const TA* __restrict__ a, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] += to_f<TA>(a[i]);
}

extern "C" int tb_residual_add(float* h, const void* a, int a_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    TB_DISPATCH_1(a_dtype, TA, tb_launch(add_kernel<TA>, dim3(blocks), dim3(256), 0, stream, h, (const TA*)a, (size_t)n));
    return tb_launch_status();
}

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

// Four consecutive elements at a time (one 16-byte or 8-byte access) when the row width allows.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float* f) {
        const float4 v = *(const float4*)p; f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* f) { *(float4*)p = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float* f) {
        const uint2 v = *(const uint2*)p;
        f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
        f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(bf16* p, const float* f) {
        __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
        *(uint2*)p = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
    }
};

// Element(s) at `p` summed over n_splits partial sums, in split order.  The loads of up to four splits are
// issued before the first addition, so their latencies overlap instead of forming a chain.
template <typename TA, int VEC>
__device__ __forceinline__ void load_sum(const TA* p, int n_splits, long long split_stride, float* v) {
    if (VEC == 4) Vec4<TA>::load(p, v); else v[0] = to_f<TA>(p[0]);
    for (int s = 1; s < n_splits; s += 4) {
        float t[4][VEC];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            if (s + k < n_splits) {
                if (VEC == 4) Vec4<TA>::load(p + (size_t)(s + k) * split_stride, t[k]);
                else t[k][0] = to_f<TA>(p[(size_t)(s + k) * split_stride]);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (s + k < n_splits) {
#pragma unroll
                for (int e = 0; e < VEC; e++) v[e] += t[k][e];
            }
    }
}

// VEC = 4: width % 4 == 0 and all rows 16-byte aligned; VEC = 1: anything.
template <typename TX, typename TW, typename TO, int VEC>
__global__ void rmsnorm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               int width, float eps, float offset) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float v[4]; Vec4<TX>::load(x + base + i, v);
            ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) { float v = to_f<TX>(x[base + i]); ss += v * v; }
    }
    ss = block_sum(ss, red);
    const float r = rsqrtf(ss / (float)width + eps);
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float v[4], g[4]; Vec4<TX>::load(x + base + i, v); Vec4<TW>::load(w + i, g);
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] = v[e] * r * (offset + g[e]);
            Vec4<TO>::store(out + base + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            out[base + i] = from_f<TO>(to_f<TX>(x[base + i]) * r * (offset + to_f<TW>(w[i])));
    }
}

// h += norm_a(a); optionally out = norm_b(h).  `a` may come as n_splits partial sums (32-bit, the
// split-K output of a matrix product, [n_splits][rows][width]); they are added in split order here,
// which saves the separate reduction pass.  The row of `a` is kept in shared memory between the two
// passes over it when it fits (row_cache != 0); a thread re-reads only elements that it wrote itself.
template <typename TA, typename TW, typename TO, int VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TA* __restrict__ a, int n_splits, long long split_stride,
                                   const TW* __restrict__ wa, float eps_a, float off_a,
                                   const TW* __restrict__ wb, float eps_b, float off_b,
                                   TO* __restrict__ out, int width, int row_cache) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float row[];
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * width;
    const int step = blockDim.x * VEC;
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < width; i += step) {
        float v[VEC];
        load_sum<TA, VEC>(a + base + i, n_splits, split_stride, v);
#pragma unroll
        for (int e = 0; e < VEC; e++) { if (row_cache) row[i + e] = v[e]; ss += v[e] * v[e]; }
    }
    ss = block_sum(ss, red);
    const float ra = rsqrtf(ss / (float)width + eps_a);
    float s2 = 0.f;
    for (int i = threadIdx.x * VEC; i < width; i += step) {
        float av[VEC], hv[VEC], g[VEC];
        if (row_cache) {
#pragma unroll
            for (int e = 0; e < VEC; e++) av[e] = row[i + e];
        } else {
            load_sum<TA, VEC>(a + base + i, n_splits, split_stride, av);
        }
        if (VEC == 4) { Vec4<float>::load(h + base + i, hv); Vec4<TW>::load(wa + i, g); }
        else { hv[0] = h[base + i]; g[0] = to_f<TW>(wa[i]); }
#pragma unroll
        for (int e = 0; e < VEC; e++) {
            hv[e] = hv[e] + av[e] * ra * (off_a + g[e]);
            if (row_cache) row[i + e] = hv[e];
            s2 += hv[e] * hv[e];
        }
        if (VEC == 4) Vec4<float>::store(h + base + i, hv); else h[base + i] = hv[0];
    }
    if (out == nullptr) return;
    s2 = block_sum(s2, red);
    const float rb = rsqrtf(s2 / (float)width + eps_b);
    for (int i = threadIdx.x * VEC; i < width; i += step) {
        float hv[VEC], g[VEC];
        if (row_cache) {
#pragma unroll
            for (int e = 0; e < VEC; e++) hv[e] = row[i + e];
        } else if (VEC == 4) Vec4<float>::load(h + base + i, hv);
        else hv[0] = h[base + i];
        if (VEC == 4) Vec4<TW>::load(wb + i, g); else g[0] = to_f<TW>(wb[i]);
#pragma unroll
        for (int e = 0; e < VEC; e++) hv[e] = hv[e] * rb * (off_b + g[e]);
        if (VEC == 4) Vec4<TO>::store(out + base + i, hv); else out[base + i] = from_f<TO>(hv[0]);
    }
}

// Many rows (prefill): WPR warps per row (1 to 16, so that a lane holds at most NV groups of four columns of a row in
// registers), eight warps a block (sixteen with WPR 16).  A row's warps meet twice, for the two sums of squares,
// through shared memory; nothing else is shared.  The grid is as many blocks as the device holds at once; a block
// walks its rows and has the next row's loads under way while it works on this one (the kernel is bound by the
// latency of its loads, not by bandwidth).  32-bit branch input (one partial sum), bfloat16 weights: the engine's
// hot case.
template <typename TO, int NV, int WPR>
__global__ void __launch_bounds__(32 * (WPR > 8 ? WPR : 8))
add_rmsnorm_rows_kernel(float* __restrict__ h, const float* __restrict__ a,
                        const bf16* __restrict__ wa, float eps_a, float off_a,
                        const bf16* __restrict__ wb, float eps_b, float off_b,
                        TO* __restrict__ out, int rows, int width) {
    constexpr int WARPS = WPR > 8 ? WPR : 8;                      // warps of a block
    constexpr int RPB = WARPS / WPR;                              // rows a block holds at a time
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float part[2][2][WARPS];                           // [row parity][which norm][warp]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = warp % WPR;                                   // which piece of the row this warp holds
    const int seg = width / WPR;                                  // columns per warp (a multiple of 4)
    const int col0 = sub * seg;
    const int stride = gridDim.x * RPB;
    int row = blockIdx.x * RPB + warp / WPR;
    float v[NV][4], hv[NV][4], nv[NV][4], nhv[NV][4];
    // a block walks its rows; the next row's branch output and residual are requested before this row's are
    // waited for, so that a block always has loads under way
    auto fetch = [&](int r, float (*va)[4], float (*vh)[4]) {
        const size_t base = (size_t)r * width + col0;
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = (k * 32 + lane) * 4;
            if (r < rows && i < seg) Vec4<float>::load(a + base + i, va[k]);
        }
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = (k * 32 + lane) * 4;
            if (r < rows && i < seg) Vec4<float>::load(h + base + i, vh[k]);
        }
    };
    fetch(row, v, hv);
    for (int it = 0; row - warp / WPR < rows; row += stride, it++) {        // the same trip count in every warp
        const bool live = row < rows;
        const size_t base = (size_t)(live ? row : 0) * width + col0;
        fetch(row + stride, nv, nhv);
        float (*pt)[WARPS] = part[it & 1];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = (k * 32 + lane) * 4;
            if (live && i < seg) ss += v[k][0] * v[k][0] + v[k][1] * v[k][1] + v[k][2] * v[k][2] + v[k][3] * v[k][3];
        }
        ss = warp_sum(ss);
        if (WPR > 1) {
            if (lane == 0) pt[0][warp] = ss;
            __syncthreads();
            ss = 0.f;
#pragma unroll
            for (int w = 0; w < WPR; w++) ss += pt[0][warp - sub + w];        // the same order in every warp of the row
        }
        const float ra = rsqrtf(ss / (float)width + eps_a);
        float s2 = 0.f;
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = (k * 32 + lane) * 4;
            if (live && i < seg) {
                float g[4];
                Vec4<bf16>::load(wa + col0 + i, g);
#pragma unroll
                for (int e = 0; e < 4; e++) { v[k][e] = hv[k][e] + v[k][e] * ra * (off_a + g[e]); s2 += v[k][e] * v[k][e]; }
                Vec4<float>::store(h + base + i, v[k]);
            }
        }
        if (out != nullptr) {                                     // the same in every thread of the launch
            s2 = warp_sum(s2);
            if (WPR > 1) {
                if (lane == 0) pt[1][warp] = s2;
                __syncthreads();
                s2 = 0.f;
#pragma unroll
                for (int w = 0; w < WPR; w++) s2 += pt[1][warp - sub + w];
            }
            const float rb = rsqrtf(s2 / (float)width + eps_b);
#pragma unroll
            for (int k = 0; k < NV; k++) {
                const int i = (k * 32 + lane) * 4;
                if (live && i < seg) {
                    float g[4], y[4];
                    Vec4<bf16>::load(wb + col0 + i, g);
#pragma unroll
                    for (int e = 0; e < 4; e++) y[e] = v[k][e] * rb * (off_b + g[e]);
                    Vec4<TO>::store(out + base + i, y);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < NV; k++)
#pragma unroll
            for (int e = 0; e < 4; e++) { v[k][e] = nv[k][e]; hv[k][e] = nhv[k][e]; }
    }
}

static int norm_threads(int width, int vec) {
    int t = ((width + vec - 1) / vec + 31) / 32 * 32;      // one access per thread and pass, if a block holds it
    return t < 64 ? 64 : (t > 1024 ? 1024 : t);
}
static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

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
    const bool vec = width % 4 == 0 && aligned16(x) && aligned16(w) && aligned16(out);
    if (vec)
        DISPATCH3(x_dtype, w_dtype, out_dtype,
            tb_launch(rmsnorm_kernel<TX, TW, TO, 4>, dim3(rows), dim3(norm_threads(width, 4)), 0, stream,
                (const TX*)x, (const TW*)w, (TO*)out, width, eps, offset));
    else
        DISPATCH3(x_dtype, w_dtype, out_dtype,
            tb_launch(rmsnorm_kernel<TX, TW, TO, 1>, dim3(rows), dim3(norm_threads(width, 1)), 0, stream,
                (const TX*)x, (const TW*)w, (TO*)out, width, eps, offset));
    return tb_launch_status();
}

// The same for few rows (decoding), where the kernel's time is a chain of memory round trips, not bandwidth: a
// thread keeps its NV groups of four columns in registers, the norm weights are fetched before the dependency
// wait (they do not depend on the kernel before), and the residual row and all partial sums are requested at
// once, so that the whole kernel waits for memory about once.
template <typename TA, typename TW, typename TO, int NV>
__global__ void __launch_bounds__(1024)
add_rmsnorm_few_kernel(float* __restrict__ h, const TA* __restrict__ a, int n_splits, long long split_stride,
                       const TW* __restrict__ wa, float eps_a, float off_a,
                       const TW* __restrict__ wb, float eps_b, float off_b, TO* __restrict__ out, int width) {
    pdl_launch_dependents();
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * width;
    float ga[NV][4], gb[NV][4], hv[NV][4], av[NV][4];
#pragma unroll
    for (int v = 0; v < NV; v++) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            Vec4<TW>::load(wa + i, ga[v]);
            if (wb != nullptr) Vec4<TW>::load(wb + i, gb[v]);
        }
    }
    pdl_wait();
#pragma unroll
    for (int v = 0; v < NV; v++) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) Vec4<float>::load(h + base + i, hv[v]);
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; e++) av[v][e] = 0.f;
        if (i < width) {
            const TA* p = a + base + i;
            for (int s0 = 0; s0 < n_splits; s0 += 8) {          // eight splits requested at a time, added in order
                float t[8][4];
#pragma unroll
                for (int k = 0; k < 8; k++) if (s0 + k < n_splits) Vec4<TA>::load(p + (size_t)(s0 + k) * split_stride, t[k]);
#pragma unroll
                for (int k = 0; k < 8; k++)
                    if (s0 + k < n_splits) {
#pragma unroll
                        for (int e = 0; e < 4; e++) av[v][e] = (s0 + k == 0) ? t[k][e] : av[v][e] + t[k][e];
                    }
            }
#pragma unroll
            for (int e = 0; e < 4; e++) ss += av[v][e] * av[v][e];
        }
    }
    ss = block_sum(ss, red);
    const float ra = rsqrtf(ss / (float)width + eps_a);
    float s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
#pragma unroll
            for (int e = 0; e < 4; e++) { hv[v][e] = hv[v][e] + av[v][e] * ra * (off_a + ga[v][e]); s2 += hv[v][e] * hv[v][e]; }
            Vec4<float>::store(h + base + i, hv[v]);
        }
    }
    if (out == nullptr) return;
    s2 = block_sum(s2, red);
    const float rb = rsqrtf(s2 / (float)width + eps_b);
#pragma unroll
    for (int v = 0; v < NV; v++) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; e++) o[e] = hv[v][e] * rb * (off_b + gb[v][e]);
            Vec4<TO>::store(out + base + i, o);
        }
    }
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
    const bool vec = width % 4 == 0 && split_stride % 4 == 0 && aligned16(h) && aligned16(a) && aligned16(wa) &&
                     aligned16(wb) && aligned16(out);
    if (vec && rows >= 64 && n_splits == 1 && a_dtype == TB_F32 && w_dtype == TB_BF16 && width <= 16 * 512) {
        // warps per row: as few as keep a lane's share of the row within four groups of four columns (it holds two
        // rows at a time: the one it works on and the one it has requested)
        int wpr = width <= 512 ? 1 : width <= 1024 ? 2 : width <= 2048 ? 4 : width <= 4096 ? 8 : 16;
        while (wpr > 1 && width % (wpr * 4)) wpr /= 2;
        const int nv = (width / wpr / 4 + 31) / 32;
        if (nv <= 4) {
            static int sms = 0;
            if (!sms) {
                int dev = 0; cudaGetDevice(&dev);
                cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
                if (sms <= 0) sms = 148;
            }
            const int rpb = (wpr > 8 ? wpr : 8) / wpr;
            const unsigned need = (unsigned)((rows + rpb - 1) / rpb);
            const unsigned threads = 32 * (wpr > 8 ? wpr : 8);
            unsigned blocks = 0;
#define ROWS(NV_, WPR_)                                                                                            \
            do {                                                                                                   \
                static int per_sm = 0;                        /* blocks of this kernel that an SM holds at once */   \
                if (!per_sm) {                                                                                     \
                    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, add_rmsnorm_rows_kernel<bf16, NV_, WPR_>, \
                                                                      (int)threads, 0) != cudaSuccess || per_sm < 1) { \
                        cudaGetLastError(); per_sm = 1;                                                            \
                    }                                                                                              \
                }                                                                                                  \
                blocks = need < (unsigned)(sms * per_sm) ? need : (unsigned)(sms * per_sm);                        \
                if (out_dtype == TB_BF16) tb_launch(add_rmsnorm_rows_kernel<bf16, NV_, WPR_>, dim3(blocks), dim3(threads), 0, stream, \
                    h, (const float*)a, (const bf16*)wa, eps_a, off_a, (const bf16*)wb, eps_b, off_b, (bf16*)out, rows, width); \
                else tb_launch(add_rmsnorm_rows_kernel<float, NV_, WPR_>, dim3(blocks), dim3(threads), 0, stream,    \
                    h, (const float*)a, (const bf16*)wa, eps_a, off_a, (const bf16*)wb, eps_b, off_b, (float*)out, rows, width); \
            } while (0)
#define ROWS_W(NV_) do { if (wpr == 1) ROWS(NV_, 1); else if (wpr == 2) ROWS(NV_, 2); else if (wpr == 4) ROWS(NV_, 4); \
                         else if (wpr == 8) ROWS(NV_, 8); else ROWS(NV_, 16); } while (0)
            if (nv <= 2) ROWS_W(2); else if (nv == 3) ROWS_W(3); else ROWS_W(4);
#undef ROWS_W
#undef ROWS
            return tb_launch_status();
        }
    }
    if (vec && rows < 64 && width <= 4 * 1024 * 4) {
        // few rows: one pass with everything in registers; as many threads as the row has groups of four
        // (measured faster than half as many threads with two groups each)
        const int groups = width / 4;
        const int nv = groups <= 1024 ? 1 : groups <= 2048 ? 2 : 4;
        const int threads = ((groups + nv - 1) / nv + 31) / 32 * 32;
#define FEW(NV_)                                                                                                   \
        DISPATCH3(a_dtype, w_dtype, out_dtype,                                                                     \
            tb_launch(add_rmsnorm_few_kernel<TX, TW, TO, NV_>, dim3(rows), dim3(threads), 0, stream,               \
                h, (const TX*)a, n_splits, split_stride, (const TW*)wa, eps_a, off_a, (const TW*)wb, eps_b, off_b, \
                (TO*)out, width))
        if (nv == 1) FEW(1); else if (nv == 2) FEW(2); else FEW(4);
#undef FEW
        return tb_launch_status();
    }
    if (vec)
        DISPATCH3(a_dtype, w_dtype, out_dtype,
            tb_launch(add_rmsnorm_kernel<TX, TW, TO, 4>, dim3(rows), dim3(norm_threads(width, 4)), smem, stream,
                h, (const TX*)a, n_splits, split_stride, (const TW*)wa, eps_a, off_a, (const TW*)wb, eps_b, off_b,
                (TO*)out, width, row_cache));
    else
        DISPATCH3(a_dtype, w_dtype, out_dtype,
            tb_launch(add_rmsnorm_kernel<TX, TW, TO, 1>, dim3(rows), dim3(norm_threads(width, 1)), smem, stream,
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

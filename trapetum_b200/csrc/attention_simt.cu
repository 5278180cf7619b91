// Attention for any head size, on the 32-bit FMA pipe: the kernels of the true
// 32-bit path and the fallback of the bfloat16 path for head sizes the
// tensor-core kernels do not take.
//
// Per query i and key j of the same sequence (runtime/cuda/codebook_gemv.cu:240-270
// is the reference's one-query form):
//   s = (q_i . k_j) * scale;  if cap: s = cap*tanh(s/cap);
//   visible(i, j) = j <= i and (window == 0 or i - j < window);
//   p = softmax over visible j (running max subtracted);  o_i = sum_j p_ij v_j
// with query head h reading kv head h / (n_heads / n_kv_heads).  Dot products,
// cap, softmax and the weighted sum are 32-bit.  The reference takes
// scale = rsqrt(head_dim) (codebook_gemv.cu:250); here scale is an argument.
//
//   tb_attn_prefill_simt  queries and keys are the step's own packed tokens
//   tb_attn_decode_simt   one query per sequence, keys from the paged cache,
//                         the key range cut into splits; partial (max, sum, o)
//                         per split go to scratch and tb_attn_combine folds them
//                         in split order (no atomics: the result is reproducible)
//
// A warp owns one (query, head); its lanes take 32 keys at a time, one key per
// lane for the dot product, then one slice of the head's dims per lane for p.v.
#include "common.cuh"

TB_EXPORT_ERROR()

__device__ __forceinline__ bool visible(int i, int j, int window) {
    return j <= i && (window <= 0 || i - j < window);
}

// Running softmax state of one warp for one (query, head).
template <int NC>
struct WarpAcc {
    float m, l;
    float o[NC];                     // dims lane, lane+32, ...
    __device__ void init() {
        m = -INFINITY; l = 0.f;
#pragma unroll
        for (int c = 0; c < NC; c++) o[c] = 0.f;
    }
};

// One chunk of up to 32 keys: lane `lane` holds the score of its key (or -inf).
// krow/vrow: pointer to that lane's key/value row (head_dim elements) or null.
template <typename T, int NC>
__device__ __forceinline__ void warp_chunk(WarpAcc<NC>& acc, const float* q_s, const T* krow, const T* vrow,
                                           bool valid, int hd, float scale, float cap, int lane) {
    float s = -INFINITY;
    if (valid) {
        float d = 0.f;
        for (int e = 0; e < hd; e++) d = fmaf(q_s[e], to_f<T>(krow[e]), d);
        s = d * scale;
        if (cap > 0.f) s = softcap_f(s, cap);
    }
    const float cm = warp_max(s);
    if (cm == -INFINITY) return;     // the whole chunk is masked
    const float m_new = fmaxf(acc.m, cm);
    const float corr = (acc.m == -INFINITY) ? 0.f : expf(acc.m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    acc.l = acc.l * corr + warp_sum(p);
    acc.m = m_new;
#pragma unroll
    for (int c = 0; c < NC; c++) acc.o[c] *= corr;
    for (int jj = 0; jj < 32; jj++) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)vrow, jj);
        if (pj == 0.f) continue;     // uniform across the warp
        const T* v = (const T*)(uintptr_t)vp;
#pragma unroll
        for (int c = 0; c < NC; c++) {
            const int d = lane + 32 * c;
            if (d < hd) acc.o[c] = fmaf(pj, to_f<T>(v[d]), acc.o[c]);
        }
    }
}

// ---------------------------------------------------------------------------
// Prefill: packed tokens, causal within each sequence.
// ---------------------------------------------------------------------------
template <typename T, int NC>
__global__ void attn_prefill_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                         long long q_stride, long long kv_stride,
                                         const int* __restrict__ seq_start, const int* __restrict__ token_seq,
                                         T* __restrict__ out, int n_tokens, int n_heads, int n_kv_heads, int hd,
                                         float scale, float cap, int window) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item % n_heads);
    const int kvh = h / (n_heads / n_kv_heads);
    const int b = token_seq[t];
    const int s0 = seq_start[b];
    const int i = t - s0;                                  // position of the query in its sequence
    float* q_s = smem + (size_t)warp * hd;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int e = lane; e < hd; e += 32) q_s[e] = to_f<T>(qrow[e]);
    __syncwarp();

    WarpAcc<NC> acc; acc.init();
    const int lo = (window > 0 && i - window + 1 > 0) ? i - window + 1 : 0;
    for (int j0 = lo; j0 <= i; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = visible(i, j, window);
        const T* krow = k + (size_t)(s0 + j) * kv_stride + (size_t)kvh * hd;
        const T* vrow = v + (size_t)(s0 + j) * kv_stride + (size_t)kvh * hd;
        warp_chunk<T, NC>(acc, q_s, valid ? krow : nullptr, valid ? vrow : nullptr, valid, hd, scale, cap, lane);
    }
    const float inv = 1.f / acc.l;
    T* orow = out + ((size_t)t * n_heads + h) * hd;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int d = lane + 32 * c;
        if (d < hd) orow[d] = from_f<T>(acc.o[c] * inv);
    }
}

// ---------------------------------------------------------------------------
// Decode: one query per sequence, keys from the paged cache.
// ---------------------------------------------------------------------------
#include "decode_args.h"

template <typename T, int NC>
__global__ void attn_decode_simt_kernel(DecodeArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int hd = a.hd;
    const int kvh = h / (a.n_heads / a.n_kv_heads);
    float* q_s = smem;                                      // [hd]
    float* red = smem + hd;                                 // [nwarp][hd + 2]
    const T* qrow = (const T*)a.q + (size_t)b * a.q_stride + (size_t)h * hd;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) q_s[e] = to_f<T>(qrow[e]);
    __syncthreads();

    const int len = a.len_after[b];
    const int i = len - 1;                                  // the query's position
    const int lo = (a.window > 0 && len - a.window > 0) ? len - a.window : 0;
    int per = (len - lo + a.n_splits - 1) / a.n_splits;
    per = (per + 31) & ~31;
    const int beg = lo + split * per;
    const int end = min(len, beg + per);

    WarpAcc<NC> acc; acc.init();
    const int* pt = a.page_table + (size_t)b * a.pt_stride;
    for (int j0 = beg + warp * 32; j0 < end; j0 += nwarp * 32) {
        const int j = j0 + lane;
        const bool valid = j < end && visible(i, j, a.window);
        const T* krow = nullptr; const T* vrow = nullptr;
        if (valid) {
            const int r = a.ring_rows > 0 ? j % a.ring_rows : j;
            const int page = pt[r / a.page_rows];
            const size_t off = (((size_t)page * a.n_kv_heads + kvh) * a.page_rows + (r % a.page_rows)) * hd;
            krow = (const T*)a.k_pool + off;
            vrow = (const T*)a.v_pool + off;
        }
        warp_chunk<T, NC>(acc, q_s, krow, vrow, valid, hd, a.scale, a.cap, lane);
    }
    // fold the warps in warp order
    float* mine = red + (size_t)warp * (hd + 2);
    if (lane == 0) { mine[hd] = acc.m; mine[hd + 1] = acc.l; }
#pragma unroll
    for (int c = 0; c < NC; c++) { const int d = lane + 32 * c; if (d < hd) mine[d] = acc.o[c]; }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < nwarp; w++) M = fmaxf(M, red[(size_t)w * (hd + 2) + hd]);
    float L = 0.f;
    for (int w = 0; w < nwarp; w++) {
        const float mw = red[(size_t)w * (hd + 2) + hd];
        if (mw != -INFINITY) L += red[(size_t)w * (hd + 2) + hd + 1] * expf(mw - M);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < nwarp; w++) {
            const float mw = red[(size_t)w * (hd + 2) + hd];
            if (mw != -INFINITY) o += red[(size_t)w * (hd + 2) + d] * expf(mw - M);
        }
        if (a.n_splits == 1) {
            ((T*)a.out)[((size_t)b * a.n_heads + h) * hd + d] = from_f<T>(o / L);
        } else {
            a.partial[(((size_t)b * a.n_heads + h) * a.n_splits + split) * (hd + 2) + d] = o;
        }
    }
    if (a.n_splits > 1 && threadIdx.x == 0) {
        float* p = a.partial + (((size_t)b * a.n_heads + h) * a.n_splits + split) * (hd + 2);
        p[hd] = M; p[hd + 1] = L;
    }
}

// out[b,h,:] = sum_s e^(m_s - M) o_s / sum_s e^(m_s - M) l_s, splits in ascending order.
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                    int n_splits, int hd) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t bh = blockIdx.x;
    const float* p = partial + bh * n_splits * (hd + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, p[(size_t)s * (hd + 2) + hd]);
    float L = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = p[(size_t)s * (hd + 2) + hd];
        if (ms != -INFINITY) L += p[(size_t)s * (hd + 2) + hd + 1] * expf(ms - M);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float ms = p[(size_t)s * (hd + 2) + hd];
            if (ms != -INFINITY) o += p[(size_t)s * (hd + 2) + d] * expf(ms - M);
        }
        out[bh * hd + d] = from_f<T>(o / L);
    }
}

static int pick_nc(int hd) {
    const int need = (hd + 31) / 32;
    int nc = 1;
    while (nc < need) nc <<= 1;
    return nc;
}

#define DISPATCH_NC(nc, ...)                                        \
    switch (nc) {                                                   \
    case 1: { constexpr int NC = 1; __VA_ARGS__; } break;           \
    case 2: { constexpr int NC = 2; __VA_ARGS__; } break;           \
    case 4: { constexpr int NC = 4; __VA_ARGS__; } break;           \
    case 8: { constexpr int NC = 8; __VA_ARGS__; } break;           \
    case 16: { constexpr int NC = 16; __VA_ARGS__; } break;         \
    default: return tb_refuse("attention: head_dim %d is larger than 512", hd); \
    }

static int check_heads(int n_heads, int n_kv_heads, int hd) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        return tb_refuse("attention: %d heads cannot share %d kv heads", n_heads, n_kv_heads);
    if (hd <= 0 || hd > 512) return tb_refuse("attention: head_dim %d is outside [1, 512]", hd);
    return 0;
}

extern "C" int tb_attn_prefill_simt(const void* q, const void* k, const void* v, long long q_stride,
                                    long long kv_stride, const int* seq_start, const int* token_seq, void* out,
                                    int dtype, int n_tokens, int n_heads, int n_kv_heads, int hd,
                                    float scale, float cap, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (check_heads(n_heads, n_kv_heads, hd)) return -1;
    const int warps = 4;
    const long long items = (long long)n_tokens * n_heads;
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * hd * sizeof(float);
    const int nc = pick_nc(hd);
    TB_DISPATCH_1(dtype, T, DISPATCH_NC(nc,
        tb_launch(attn_prefill_simt_kernel<T, NC>, dim3(blocks), dim3(warps * 32), smem, stream, 
            (const T*)q, (const T*)k, (const T*)v, q_stride, kv_stride, seq_start, token_seq, (T*)out,
            n_tokens, n_heads, n_kv_heads, hd, scale, cap, window)));
    return tb_launch_status();
}

extern "C" long long tb_attn_decode_scratch_floats(int batch, int n_heads, int hd, int n_splits) {
    return n_splits > 1 ? (long long)batch * n_heads * n_splits * (hd + 2) : 0;
}

extern "C" int tb_attn_decode_simt(const DecodeArgs* args, int dtype, int batch, cudaStream_t stream) {
    if (batch <= 0) return 0;
    DecodeArgs a = *args;
    const int hd = a.hd;
    if (check_heads(a.n_heads, a.n_kv_heads, hd)) return -1;
    if (a.n_splits < 1 || a.n_splits > 65535) return tb_refuse("attention: n_splits=%d", a.n_splits);
    if (a.n_heads > 65535) return tb_refuse("attention: %d heads is more than one launch takes", a.n_heads);
    if (a.n_splits > 1 && a.partial == nullptr) return tb_refuse("attention: splits need scratch");
    if (a.page_rows <= 0 || (a.ring_rows > 0 && a.ring_rows % a.page_rows))
        return tb_refuse("attention: page_rows=%d ring_rows=%d", a.page_rows, a.ring_rows);
    if (a.ring_rows > 0 && (a.window <= 0 || a.window > a.ring_rows))
        return tb_refuse("attention: a ring of %d rows cannot hold a window of %d", a.ring_rows, a.window);
    const int warps = 4;
    const size_t smem = ((size_t)hd + (size_t)warps * (hd + 2)) * sizeof(float);
    dim3 grid(batch, a.n_heads, a.n_splits);
    const int nc = pick_nc(hd);
    TB_DISPATCH_1(dtype, T, DISPATCH_NC(nc,
        tb_launch(attn_decode_simt_kernel<T, NC>, dim3(grid), dim3(warps * 32), smem, stream, a)));
    int st = tb_launch_status();
    if (st) return st;
    if (a.n_splits > 1) {
        const unsigned rows = (unsigned)batch * a.n_heads;
        TB_DISPATCH_1(dtype, T,
            tb_launch(attn_combine_kernel<T>, dim3(rows), dim3(128), 0, stream, a.partial, (T*)a.out, a.n_splits, hd));
        st = tb_launch_status();
    }
    return st;
}

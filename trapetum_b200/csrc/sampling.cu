// Choosing the next token from 32-bit logits, on the device.
//
//   tb_argmax  greedy: the largest logit, the smallest index on a tie.  Two stages
//              like the reference's argmax_stage1/2 (runtime/cuda/codebook_gemv.cu:544-591),
//              but for many rows at once; stage 1 writes (value, index) per chunk
//              to scratch, stage 2 folds the chunks in order.
//   tb_sample  what the reference's server does on the host (runtime/src/bin/serve.rs:41-72,
//              285-294), per row and in this order:
//                1. repetition penalty over the row's recent tokens, each distinct id
//                   once: logit > 0 ? logit / penalty : logit * penalty  (off if <= 1)
//                2. temperature <= 0: argmax.  Otherwise p_i ~ exp((l_i - max) / T)
//                3. nucleus: the smallest set of most probable tokens whose mass
//                   reaches top_p (all tokens if top_p >= 1)
//                4. a draw u in [0,1), given by the caller, picks the token at which
//                   the running sum of kept p_i, taken in index order, passes
//                   u * (kept mass)
//              The reference sorts and keeps the 256 largest logits before step 3
//              and walks them in sorted order; the kept set is the same whenever
//              the nucleus has at most 256 tokens, and the distribution of the
//              draw is the same.  Its draw comes from a xorshift seeded by the
//              wall clock; here the caller owns the generator, so a run repeats.
//
// All sums are 32-bit and taken in a fixed order.
#include "common.cuh"

TB_EXPORT_ERROR()

#define ARGMAX_CHUNK 8192

struct ValIdx { float v; int i; };

__device__ __forceinline__ ValIdx better(ValIdx a, ValIdx b) {
    // NaN never wins; ties go to the smaller index
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ValIdx block_best(ValIdx x, ValIdx* red /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ValIdx y; y.v = __shfl_xor_sync(0xffffffffu, x.v, o); y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) red[warp] = x;
    __syncthreads();
    ValIdx t; t.v = -INFINITY; t.i = 0x7fffffff;
    if (lane < nwarp) t = red[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ValIdx y; y.v = __shfl_xor_sync(0xffffffffu, t.v, o); y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
        t = better(t, y);
    }
    return t;
}

__global__ void argmax_stage1_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                                     float* __restrict__ pval, int* __restrict__ pidx, int n_chunks) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ ValIdx red[32];
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    const int beg = chunk * ARGMAX_CHUNK, end = min(vocab, beg + ARGMAX_CHUNK);
    ValIdx b; b.v = -INFINITY; b.i = 0x7fffffff;
    for (int i = beg + threadIdx.x; i < end; i += blockDim.x) { ValIdx c; c.v = x[i]; c.i = i; b = better(b, c); }
    b = block_best(b, red);
    if (threadIdx.x == 0) { pval[(size_t)row * n_chunks + chunk] = b.v; pidx[(size_t)row * n_chunks + chunk] = b.i; }
}

__global__ void argmax_stage2_kernel(const float* __restrict__ pval, const int* __restrict__ pidx,
                                     int n_chunks, int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ ValIdx red[32];
    const int row = blockIdx.x;
    ValIdx b; b.v = -INFINITY; b.i = 0x7fffffff;
    for (int i = threadIdx.x; i < n_chunks; i += blockDim.x) {
        ValIdx c; c.v = pval[(size_t)row * n_chunks + i]; c.i = pidx[(size_t)row * n_chunks + i];
        b = better(b, c);
    }
    b = block_best(b, red);
    if (threadIdx.x == 0) out[row] = (b.i == 0x7fffffff) ? 0 : b.i;
}

extern "C" long long tb_argmax_scratch_bytes(int rows, int vocab) {
    const long long chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    return (long long)rows * chunks * 8;
}

extern "C" int tb_argmax(const float* logits, long long row_stride, int rows, int vocab, int* out,
                         void* scratch, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return tb_refuse("argmax: vocab=%d", vocab);
    if (rows > 65535) return tb_refuse("argmax: %d rows is more than one call takes", rows);
    const int n_chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    float* pval = (float*)scratch;
    int* pidx = (int*)(pval + (size_t)rows * n_chunks);
    dim3 grid(n_chunks, rows);
    tb_launch(argmax_stage1_kernel, dim3(grid), dim3(256), 0, stream, logits, row_stride, vocab, pval, pidx, n_chunks);
    tb_launch(argmax_stage2_kernel, dim3(rows), dim3(128), 0, stream, pval, pidx, n_chunks, out);
    return tb_launch_status();
}

// ---------------------------------------------------------------------------
// Sampling: one CTA per row.
// ---------------------------------------------------------------------------

// Floats as unsigned keys whose order is the floats' order.
__device__ __forceinline__ unsigned f2key(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct SampleArgs {
    float* logits; long long row_stride; int vocab;
    const float* temperature;      // [rows]
    const float* top_p;            // [rows]
    const float* penalty;          // [rows]
    const float* draw;             // [rows] u in [0,1)
    const int* recent; int n_recent;   // [rows, n_recent] recent token ids, -1 = none
    int* out;                      // [rows]
};

__global__ void __launch_bounds__(1024) sample_kernel(SampleArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    __shared__ ValIdx redvi[32];
    __shared__ float scan[1024];
    __shared__ int chosen;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    float* x = a.logits + (size_t)row * a.row_stride;
    const int V = a.vocab;

    // 1. repetition penalty, each distinct recent id once
    const float pen = a.penalty ? a.penalty[row] : 1.f;
    if (pen > 1.f && a.recent) {
        const int* rec = a.recent + (size_t)row * a.n_recent;
        for (int j = tid; j < a.n_recent; j += nt) {
            const int id = rec[j];
            if (id < 0 || id >= V) continue;
            bool first = true;
            for (int k = 0; k < j; k++) if (rec[k] == id) { first = false; break; }
            if (first) { const float l = x[id]; x[id] = l > 0.f ? l / pen : l * pen; }
        }
        __syncthreads();
    }

    // 2. greedy
    const float T = a.temperature ? a.temperature[row] : 0.f;
    if (!(T > 0.f)) {
        ValIdx b; b.v = -INFINITY; b.i = 0x7fffffff;
        for (int i = tid; i < V; i += nt) { ValIdx c; c.v = x[i]; c.i = i; b = better(b, c); }
        b = block_best(b, redvi);
        if (tid == 0) a.out[row] = (b.i == 0x7fffffff) ? 0 : b.i;
        return;
    }

    float mx = -INFINITY;
    for (int i = tid; i < V; i += nt) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, red);
    const float invT = 1.f / T;
    float z = 0.f;
    for (int i = tid; i < V; i += nt) z += expf((x[i] - mx) * invT);
    z = block_sum(z, red);

    // 3. nucleus: the largest threshold key whose mass still reaches top_p * z
    const float top_p = a.top_p ? a.top_p[row] : 1.f;
    unsigned thr = 0u;                               // keep everything
    float kept = z;
    if (top_p < 1.f) {
        const float want = top_p * z;
        unsigned lo = 0u;                            // mass(lo) >= want always holds
        for (int bit = 31; bit >= 0; bit--) {
            const unsigned cand = lo | (1u << bit);
            float s = 0.f;
            for (int i = tid; i < V; i += nt) { const float l = x[i]; if (f2key(l) >= cand) s += expf((l - mx) * invT); }
            s = block_sum(s, red);
            if (s >= want) { lo = cand; kept = s; }
        }
        thr = lo;
    }

    // 4. inverse CDF over the kept tokens in index order
    const float target = a.draw[row] * kept;
    const int per = (V + nt - 1) / nt;
    const int beg = min(V, tid * per), end = min(V, beg + per);
    float mine = 0.f;
    for (int i = beg; i < end; i++) { const float l = x[i]; if (f2key(l) >= thr) mine += expf((l - mx) * invT); }
    scan[tid] = mine;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {                                   // serial prefix over 1024 partial sums: fixed order
        float run = 0.f;
        for (int t = 0; t < nt; t++) { const float v = scan[t]; scan[t] = run; run += v; }
    }
    __syncthreads();
    const float before = scan[tid];
    if (mine > 0.f && target >= before && target < before + mine) {
        float run = before; int pick = -1;
        for (int i = beg; i < end; i++) {
            const float l = x[i];
            if (f2key(l) >= thr) { run += expf((l - mx) * invT); pick = i; if (target < run) break; }
        }
        chosen = pick;
    }
    __syncthreads();
    if (chosen < 0) {
        // the draw fell past the last partial sum through rounding: take the last kept token
        ValIdx b; b.v = -INFINITY; b.i = 0x7fffffff;
        for (int i = tid; i < V; i += nt) if (f2key(x[i]) >= thr) { ValIdx c; c.v = (float)i; c.i = -i; b = better(b, c); }
        b = block_best(b, redvi);
        if (tid == 0) chosen = (b.i == 0x7fffffff) ? 0 : -b.i;
        __syncthreads();
    }
    if (tid == 0) a.out[row] = chosen;
}

extern "C" int tb_sample(const SampleArgs* args, int rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    SampleArgs a = *args;
    if (a.vocab <= 0) return tb_refuse("sample: vocab=%d", a.vocab);
    if (a.draw == nullptr) return tb_refuse("sample: the draws are missing");
    tb_launch(sample_kernel, dim3(rows), dim3(1024), 0, stream, a);
    return tb_launch_status();
}

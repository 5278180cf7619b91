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

// ---------------------------------------------------------------------------
// Sampling over a large vocabulary: the same four steps, but a row's elements are spread over many CTAs and
// every pass over the row is one launch of (chunks x rows) CTAs, so that a row of 256,000 logits is read at the
// speed of the whole GPU and not of one SM (the one-CTA kernel above takes 1.7 ms for such rows with a nucleus,
// most of a decode step).
//
// Masses are fixed-point: m_i = round(2^32 e^((l_i - max) / T)), summed in 64-bit integers.  Integer sums do not
// depend on their order, so histograms can be built with atomics and the draw still repeats bit for bit.
// The nucleus threshold is found by a radix search on the order-preserving key of the logit: three passes
// (11 + 11 + 10 bits), each a histogram of mass per digit among the elements that match the digits found so far,
// and a scan from the top for the digit at which the mass above reaches top_p x total.
//
//   sample_chunk_max  per chunk: repetition penalty on the chunk's ids, then (max, index)   [also the greedy choice];
//                     clears the row's histograms
//   sample_hist<R>    per chunk: (R > 0: first the digit of pass R-1, found by every CTA for itself from the
//                     finished histogram;) mass histogram of pass R            [rows with a nucleus only]
//   sample_chunk_mass per chunk: the last digit, hence the threshold; mass of the chunk's kept elements
//   sample_pick       per row: target = u x kept mass; the chunk and then the element at which the running sum
//                     of kept masses, in index order, passes the target
// ---------------------------------------------------------------------------
#define S_CHUNK 8192
#define S_BINS 2048
typedef unsigned long long u64;

struct SampleState {              // per row
    u64 mass_above;               // mass of the elements above the digits found so far
    u64 want;                     // top_p x total mass
    unsigned prefix;              // the digits found so far (the high bits of the threshold key)
    int nucleus;                  // 1: this row searches a threshold; 0: keeps everything (or is greedy)
};

struct SampleWide {
    SampleArgs a;
    int n_chunks;
    float* pmax; int* pidx;       // [rows][n_chunks]
    u64* hist;                    // [rows][3][S_BINS]
    u64* cmass;                   // [rows][n_chunks]
    SampleState* state;           // [rows][3]: after pass 0, 1, 2
};

__device__ __forceinline__ u64 fixed_mass(float l, float mx, float invT) {
    return __float2ull_rn(expf((l - mx) * invT) * 4294967296.0f);
}
// the row's maximum from the chunk maxima (every thread of the CTA gets it)
__device__ __forceinline__ float row_max(const SampleWide& w, int row, float* red /* 33 */) {
    float m = -INFINITY;
    for (int c = threadIdx.x; c < w.n_chunks; c += blockDim.x) m = fmaxf(m, w.pmax[(size_t)row * w.n_chunks + c]);
    return block_max(m, red);
}

__global__ void __launch_bounds__(256) sample_chunk_max_kernel(SampleWide w) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ ValIdx red[32];
    __shared__ int rec_s[1024];
    const int row = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
    const SampleArgs& a = w.a;
    float* x = a.logits + (size_t)row * a.row_stride;
    const int beg = chunk * S_CHUNK, end = min(a.vocab, beg + S_CHUNK);
    // this CTA's share of the row's histograms starts at zero
    for (int i = chunk * 256 + tid; i < 3 * S_BINS; i += gridDim.x * 256) w.hist[(size_t)row * 3 * S_BINS + i] = 0ull;
    // repetition penalty, each distinct recent id once; a CTA sees to the ids of its own chunk
    const float pen = a.penalty ? a.penalty[row] : 1.f;
    if (pen > 1.f && a.recent) {
        const int* rec = a.recent + (size_t)row * a.n_recent;
        for (int j0 = 0; j0 < a.n_recent; j0 += 1024) {            // (lists longer than 1024 in pieces; each id is
            const int n = min(1024, a.n_recent - j0);               //  compared with the whole list before it)
            __syncthreads();
            for (int j = tid; j < n; j += 256) rec_s[j] = rec[j0 + j];
            __syncthreads();
            for (int j = tid; j < n; j += 256) {
                const int id = rec_s[j];
                if (id < beg || id >= end) continue;
                bool first = true;
                for (int k = 0; k < j && first; k++) first = rec_s[k] != id;
                for (int k = 0; k < j0 && first; k++) first = rec[k] != id;
                if (first) { const float l = x[id]; x[id] = l > 0.f ? l / pen : l * pen; }
            }
        }
        __syncthreads();
    }
    ValIdx b; b.v = -INFINITY; b.i = 0x7fffffff;
    for (int i = beg + tid; i < end; i += 256) { ValIdx c; c.v = x[i]; c.i = i; b = better(b, c); }
    b = block_best(b, red);
    if (tid == 0) { w.pmax[(size_t)row * w.n_chunks + chunk] = b.v; w.pidx[(size_t)row * w.n_chunks + chunk] = b.i; }
}

// the digit of pass R of a key, and whether the key matches the digits found before it
template <int R> __device__ __forceinline__ bool digit_of(unsigned key, unsigned prefix, int& bin) {
    if (R == 0) { bin = key >> 21; return true; }
    if (R == 1) { bin = (key >> 10) & 2047; return (key >> 21) == prefix; }
    bin = key & 1023; return (key >> 10) == prefix;
}

// The digit of pass R from its finished histogram `g` (in shared memory), by a CTA of 256 threads: each thread sums
// eight digits, warp 0 scans the sums from the top, and the lane in which the mass above reaches `want` walks down
// its own sums and then the eight digits of one of them.  `*st` (shared memory) is the state before the pass on
// entry and the state after it on return.
template <int R>
__device__ void select_digit(const u64* g, u64* part /* 256 */, SampleState* st_io, float top_p) {
    const int tid = threadIdx.x, lane = tid & 31;
    u64 s = 0ull;
#pragma unroll
    for (int k = 0; k < 8; k++) s += g[tid * 8 + k];
    part[tid] = s;
    __syncthreads();
    if (tid < 32) {
        SampleState st = *st_io;
        u64 mine = 0ull;
#pragma unroll
        for (int k = 0; k < 8; k++) mine += part[lane * 8 + k];
        u64 incl = mine;                             // this lane's sum and those of the lanes above it (higher digits)
        for (int o = 1; o < 32; o <<= 1) { const u64 v = __shfl_down_sync(0xffffffffu, incl, o); if (lane + o < 32) incl += v; }
        if (R == 0) {
            const u64 tot = __shfl_sync(0xffffffffu, incl, 0);       // the total mass, and what the nucleus has to reach
            const double want = (double)top_p * (double)tot;
            st.want = want < 1.0 ? 1ull : (u64)want;
            if (st.want > tot) st.want = tot;
        }
        const u64 above = st.mass_above + incl - mine;
        const bool here = above < st.want && above + mine >= st.want;
        u64 acc = above;
        int b = 0;
        if (here) {
            int t = lane * 8 + 7;
            for (; t > lane * 8; t--) { if (acc + part[t] >= st.want) break; acc += part[t]; }
            b = t * 8 + 7;
            for (; b > t * 8; b--) { if (acc + g[b] >= st.want) break; acc += g[b]; }
        }
        const unsigned who = __ballot_sync(0xffffffffu, here);
        const int src = who ? __ffs(who) - 1 : 0;    // (exactly one lane, unless the masses are all zero)
        st.mass_above = __shfl_sync(0xffffffffu, acc, src);
        b = __shfl_sync(0xffffffffu, b, src);
        st.prefix = (R == 0) ? (unsigned)b : (R == 1) ? ((st.prefix << 11) | (unsigned)b) : ((st.prefix << 10) | (unsigned)b);
        if (lane == 0) *st_io = st;
    }
    __syncthreads();
}

// The state before pass R for this CTA (R == 0: the start), into shared memory: found from the finished histogram
// of pass R-1; the CTA of chunk 0 also leaves it in memory for the launches after this one.  `g`: S_BINS sums.
template <int R>
__device__ void state_before_pass(const SampleWide& w, int row, u64* g, u64* part, SampleState* out) {
    if (threadIdx.x == 0) {
        SampleState st;
        if (R <= 1) {
            const float T = w.a.temperature ? w.a.temperature[row] : 0.f;
            const float tp = w.a.top_p ? w.a.top_p[row] : 1.f;
            st.mass_above = 0ull; st.want = 0ull; st.prefix = 0u; st.nucleus = (T > 0.f && tp < 1.f) ? 1 : 0;
        } else {
            st = w.state[(size_t)row * 3 + (R > 1 ? R - 2 : 0)];
        }
        *out = st;
    }
    __syncthreads();
    if constexpr (R > 0) {
        if (!out->nucleus) return;
        const u64* gg = w.hist + ((size_t)row * 3 + (R - 1)) * S_BINS;
        for (int j = threadIdx.x; j < S_BINS; j += blockDim.x) g[j] = gg[j];
        __syncthreads();
        select_digit<R - 1>(g, part, out, R == 1 ? w.a.top_p[row] : 0.f);
        if (threadIdx.x == 0 && blockIdx.x == 0) w.state[(size_t)row * 3 + (R - 1)] = *out;
    }
}

template <int R>
__global__ void __launch_bounds__(256) sample_hist_kernel(SampleWide w) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ u64 g[S_BINS];
    __shared__ u64 part[256];
    __shared__ SampleState s_st;
    __shared__ float red[33];
    const int row = blockIdx.y, chunk = blockIdx.x;
    state_before_pass<R>(w, row, g, part, &s_st);
    const SampleState st = s_st;
    if (!st.nucleus) return;
    __syncthreads();
    // A mass is at most 2^32.  Its low 16 bits and the rest are summed in two 32-bit histograms, whose atomics the
    // shared memory has natively (a 64-bit one is a compare-and-swap loop, slow where most of a row falls into a
    // few digits); a chunk's 8192 elements cannot overflow either.
    unsigned* lo = (unsigned*)g;
    unsigned* hi = lo + S_BINS;
    for (int i = threadIdx.x; i < 2 * S_BINS; i += blockDim.x) lo[i] = 0u;
    const float* x = w.a.logits + (size_t)row * w.a.row_stride;
    const float mx = row_max(w, row, red), invT = 1.f / w.a.temperature[row];   // (block_max has the barriers)
    const int beg = chunk * S_CHUNK, end = min(w.a.vocab, beg + S_CHUNK);
    for (int i = beg + threadIdx.x; i < end; i += blockDim.x) {
        const float l = x[i];
        int bin;
        if (!digit_of<R>(f2key(l), st.prefix, bin)) continue;
        const u64 m = fixed_mass(l, mx, invT);
        atomicAdd(&lo[bin], (unsigned)(m & 0xffffu));
        atomicAdd(&hi[bin], (unsigned)(m >> 16));
    }
    __syncthreads();
    u64* out = w.hist + ((size_t)row * 3 + R) * S_BINS;
    for (int i = threadIdx.x; i < S_BINS; i += blockDim.x) {
        const u64 m = (u64)lo[i] + ((u64)hi[i] << 16);
        if (m) atomicAdd(&out[i], m);
    }
}

__global__ void __launch_bounds__(256) sample_chunk_mass_kernel(SampleWide w, int nucleus) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ u64 g[S_BINS];
    __shared__ u64 part[256];
    __shared__ SampleState s_st;
    __shared__ u64 red8[8];
    __shared__ float red[33];
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float T = w.a.temperature ? w.a.temperature[row] : 0.f;
    if (!(T > 0.f)) return;
    unsigned thr = 0u;                                              // keep everything
    if (nucleus) {
        state_before_pass<3>(w, row, g, part, &s_st);
        if (s_st.nucleus) thr = s_st.prefix;                       // after the last pass the digits are the whole key
    }
    const float* x = w.a.logits + (size_t)row * w.a.row_stride;
    const float mx = row_max(w, row, red), invT = 1.f / T;
    const int beg = chunk * S_CHUNK, end = min(w.a.vocab, beg + S_CHUNK);
    u64 m = 0ull;
    for (int i = beg + threadIdx.x; i < end; i += blockDim.x) {
        const float l = x[i];
        if (f2key(l) >= thr) m += fixed_mass(l, mx, invT);
    }
    for (int o = 16; o > 0; o >>= 1) m += __shfl_xor_sync(0xffffffffu, m, o);
    if ((threadIdx.x & 31) == 0) red8[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 t = 0ull;
        for (int k = 0; k < (int)(blockDim.x >> 5); k++) t += red8[k];
        w.cmass[(size_t)row * w.n_chunks + chunk] = t;
    }
}

__global__ void __launch_bounds__(256) sample_pick_kernel(SampleWide w, int nucleus) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ u64 part[256];
    __shared__ u64 cm[256];                                          // the chunks' kept masses: read side by side
    __shared__ float red[33];
    __shared__ int s_chunk;
    __shared__ u64 s_base, s_target;
    const int row = blockIdx.x, tid = threadIdx.x;
    const SampleArgs& a = w.a;
    const float T = a.temperature ? a.temperature[row] : 0.f;
    if (!(T > 0.f)) {
        // greedy: the best of the chunk maxima, the smallest index on a tie
        if (tid == 0) {
            ValIdx b; b.v = -INFINITY; b.i = 0x7fffffff;
            for (int c = 0; c < w.n_chunks; c++) {
                ValIdx v; v.v = w.pmax[(size_t)row * w.n_chunks + c]; v.i = w.pidx[(size_t)row * w.n_chunks + c];
                b = better(b, v);
            }
            a.out[row] = (b.i == 0x7fffffff) ? 0 : b.i;
        }
        return;
    }
    unsigned thr = 0u;
    if (nucleus) { const SampleState st = w.state[(size_t)row * 3 + 2]; if (st.nucleus) thr = st.prefix; }
    for (int c = tid; c < w.n_chunks; c += 256) cm[c] = w.cmass[(size_t)row * w.n_chunks + c];
    const float mx = row_max(w, row, red);                          // (has the barriers that cm needs, too)
    if (tid == 0) {
        u64 kept = 0ull;
        for (int c = 0; c < w.n_chunks; c++) kept += cm[c];
        const double tg = (double)a.draw[row] * (double)kept;
        u64 target = (u64)tg;
        if (target >= kept) target = kept - 1;                      // (kept >= 2^32: the row's maximum has mass 2^32)
        u64 base = 0ull;
        int c = 0;
        for (; c < w.n_chunks - 1; c++) { if (base + cm[c] > target) break; base += cm[c]; }
        s_chunk = c; s_base = base; s_target = target;
    }
    __syncthreads();
    const float* x = a.logits + (size_t)row * a.row_stride;
    const float invT = 1.f / T;
    constexpr int PER = S_CHUNK / 256;                              // consecutive elements per thread: index order
    const int beg = s_chunk * S_CHUNK + tid * PER, end = min(a.vocab, beg + PER);
    u64 mine = 0ull;
    for (int i = beg; i < end; i++) { const float l = x[i]; if (f2key(l) >= thr) mine += fixed_mass(l, mx, invT); }
    part[tid] = mine;
    __syncthreads();
    if (tid < 32) {
        // exclusive prefix over 256 sums: a lane sums its 8, the lanes scan, each lane writes its 8 prefixes
        u64 loc[8], sum = 0ull;
#pragma unroll
        for (int k = 0; k < 8; k++) { loc[k] = part[tid * 8 + k]; sum += loc[k]; }
        u64 incl = sum;
        for (int o = 1; o < 32; o <<= 1) { const u64 v = __shfl_up_sync(0xffffffffu, incl, o); if (tid >= o) incl += v; }
        u64 run = s_base + incl - sum;
#pragma unroll
        for (int k = 0; k < 8; k++) { part[tid * 8 + k] = run; run += loc[k]; }
    }
    __syncthreads();
    const u64 before = part[tid], target = s_target;
    if (mine > 0ull && target >= before && target < before + mine) {
        u64 run = before; int pick = beg;
        for (int i = beg; i < end; i++) {
            const float l = x[i];
            if (f2key(l) >= thr) { run += fixed_mass(l, mx, invT); pick = i; if (target < run) break; }
        }
        a.out[row] = pick;
    }
}

extern "C" long long tb_sample_wide_scratch_bytes(int rows, int vocab) {
    const long long chunks = (vocab + S_CHUNK - 1) / S_CHUNK;
    return (long long)rows * (chunks * (4 + 4 + 8) + 3LL * S_BINS * 8 + 3LL * (long long)sizeof(SampleState)) + 256;
}

// `nucleus`: 0 if the caller knows that every row has top_p >= 1 (the threshold passes are then not launched).
extern "C" int tb_sample_wide(const SampleArgs* args, int rows, void* scratch, int nucleus, cudaStream_t stream) {
    if (rows <= 0) return 0;
    SampleWide w;
    w.a = *args;
    if (w.a.vocab <= 0) return tb_refuse("sample: vocab=%d", w.a.vocab);
    if (w.a.draw == nullptr) return tb_refuse("sample: the draws are missing");
    if (rows > 65535) return tb_refuse("sample: %d rows is more than one call takes", rows);
    if ((w.a.vocab + S_CHUNK - 1) / S_CHUNK > 256) return tb_refuse("sample: a vocabulary of %d is more than this kernel takes", w.a.vocab);
    if (scratch == nullptr || ((uintptr_t)scratch & 15)) return tb_refuse("sample: needs 16-byte aligned scratch");
    w.n_chunks = (w.a.vocab + S_CHUNK - 1) / S_CHUNK;
    char* p = (char*)scratch;
    w.hist = (u64*)p; p += (size_t)rows * 3 * S_BINS * 8;
    w.cmass = (u64*)p; p += (size_t)rows * w.n_chunks * 8;
    w.state = (SampleState*)p; p += (size_t)rows * 3 * sizeof(SampleState);
    w.pmax = (float*)p; p += (size_t)rows * w.n_chunks * 4;
    w.pidx = (int*)p;
    const dim3 per_chunk(w.n_chunks, rows);
    tb_launch(sample_chunk_max_kernel, dim3(per_chunk), dim3(256), 0, stream, w);
    if (nucleus) {
        tb_launch(sample_hist_kernel<0>, dim3(per_chunk), dim3(256), 0, stream, w);
        tb_launch(sample_hist_kernel<1>, dim3(per_chunk), dim3(256), 0, stream, w);
        tb_launch(sample_hist_kernel<2>, dim3(per_chunk), dim3(256), 0, stream, w);
    }
    tb_launch(sample_chunk_mass_kernel, dim3(per_chunk), dim3(256), 0, stream, w, nucleus);
    tb_launch(sample_pick_kernel, dim3(rows), dim3(256), 0, stream, w, nucleus);
    return tb_launch_status();
}

extern "C" int tb_sample(const SampleArgs* args, int rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    SampleArgs a = *args;
    if (a.vocab <= 0) return tb_refuse("sample: vocab=%d", a.vocab);
    if (a.draw == nullptr) return tb_refuse("sample: the draws are missing");
    tb_launch(sample_kernel, dim3(rows), dim3(1024), 0, stream, a);
    return tb_launch_status();
}

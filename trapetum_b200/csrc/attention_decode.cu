// Decode attention over the paged cache at memory speed (bfloat16).
//
// One query token per sequence; its keys and values are the sequence's pages in the
// cache.  Same formula as the reference's attn_k (runtime/cuda/codebook_gemv.cu:240-270:
// s = q.k * scale, optional cap*tanh(s/cap), softmax, sum of p*v), but where that
// kernel runs one block per head with a block-wide tree reduction per key and a
// single-thread softmax, here
//   * a CTA owns (sequence, kv head, split of the page range) and serves all query
//     heads of the group from one read of K and V;
//   * pages (64 keys x head_dim, contiguous in the pool) are brought into shared
//     memory by bulk copies of the TMA unit, several pages ahead, tracked by mbarriers;
//   * each of the 16 warps takes 4 keys of a page; a key's head_dim is spread over
//     head_dim/8 lanes (16 bytes each); partial dot products are reduced with a
//     butterfly that leaves one (key, head) score per lane, so cap, exp and the
//     running softmax are computed once per score;
//   * all math is 32-bit; splits write (max, sum, o) partials that a second kernel
//     folds in split order (no atomics).
// Rows of a page beyond the sequence's keys (or outside the window) are never used,
// not even multiplied by zero: stale or uninitialised rows cannot leak.
//
// Takes head_dim in {32, 64, 128, 256} and up to 8 query heads per kv head; other shapes are
// refused and the caller uses the generic kernel.  Two kernels live here: the scalar one described
// above (tb_attn_decode_lanes: head_dim 32, and comparison) and the tensor-core one further down
// (tb_attn_decode, tb_attn_decode_stream: the product path for head_dim 64, 128 and 256).
#include "common.cuh"
#include "async.cuh"
#include <cuda.h>

TB_EXPORT_ERROR()

#define PAGE 64

__device__ int g_attn_error = 0;          // 0, or: 1 a bounded wait ran out, 2 shared memory less aligned than budgeted, 3 too many runs in a CTA

#include "decode_args.h"

template <int HD> struct DCfg {
    static constexpr int NWARP = HD >= 64 ? 16 : 8;                  // more warps hide more latency; a warp needs
    static constexpr int KPW = PAGE / NWARP;                         // at least one pass of 256 / HD keys per page
    static constexpr int PAGE_BYTES = PAGE * HD * 2;                 // one page of K (or V) for one kv head
    static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
    static constexpr int STAGES_RAW = (192 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 128;
};

__device__ __forceinline__ void bf16x8_to_f32(const uint4& w, float* f) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

template <int HD, int G>
__global__ void __launch_bounds__(DCfg<HD>::NWARP * 32, 1) attn_decode_kernel(DecodeArgs a) {
    pdl_launch_dependents();
    using C = DCfg<HD>;
    constexpr int NWARP = C::NWARP, KPW = C::KPW;
    constexpr int LPK = HD / 8;                    // lanes per key
    constexpr int KP = 32 / LPK;                   // keys per pass of a warp
    constexpr int NP = KPW / KP;                   // passes per page
    constexpr int N = NP * G;                      // scores a lane group produces per page
    constexpr int NF = N > LPK ? N / LPK : 1;      // scores a lane holds after the butterfly
    constexpr int SPREAD = N > LPK ? 1 : LPK / N;  // lanes that hold the same score
    static_assert(KP <= KPW && NP >= 1, "head_dim too small for this kernel");

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
    __shared__ int s_abort;

    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPK, kg = lane / LPK;

    const int len = a.len_after[b];
    const int lo = (a.window > 0 && len > a.window) ? len - a.window : 0;
    // the rows of this sequence in "row space": positions, or ring rows
    int first_page, n_pages;
    if (a.ring_rows > 0) { first_page = 0; n_pages = (min(len, a.ring_rows) + PAGE - 1) / PAGE; }
    else { first_page = lo / PAGE; n_pages = (len - 1) / PAGE - first_page + 1; }
    const int per = (n_pages + a.n_splits - 1) / a.n_splits;
    const int pg_beg = first_page + split * per;
    const int pg_end = min(first_page + n_pages, pg_beg + per);
    const int n = max(0, pg_end - pg_beg);
    const int* pt = a.page_table + (size_t)b * a.pt_stride;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) mbar_init(&full[s], 1);
        s_abort = 0;
        mbar_init_fence();
    }
    __syncthreads();

    auto issue = [&](int i) {
        const int s = i % C::STAGES;
        const int page = pt[pg_beg + i];
        const size_t off = ((size_t)page * a.n_kv_heads + kvh) * PAGE * HD;
        uint8_t* dst = smem + s * C::STAGE_BYTES;
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
        bulk_load(dst, (const bf16*)a.k_pool + off, C::PAGE_BYTES, &full[s]);
        bulk_load(dst + C::PAGE_BYTES, (const bf16*)a.v_pool + off, C::PAGE_BYTES, &full[s]);
    };
    pdl_wait();                                     // the cache rows of this step and q come from earlier kernels
    if (threadIdx.x == 0)
        for (int i = 0; i < n && i < C::STAGES; i++) issue(i);

    // this lane's slice of the queries, already multiplied by the scale
    float q[G][8];
#pragma unroll
    for (int g = 0; g < G; g++) {
        const bf16* qp = (const bf16*)a.q + (size_t)b * a.q_stride + (size_t)(kvh * G + g) * HD + sub * 8;
        float f[8];
        bf16x8_to_f32(*(const uint4*)qp, f);
#pragma unroll
        for (int e = 0; e < 8; e++) q[g][e] = f[e] * a.scale;
    }

    float m[G], o[G][8], l_lane[NF];
#pragma unroll
    for (int g = 0; g < G; g++) {
        m[g] = -INFINITY;
#pragma unroll
        for (int e = 0; e < 8; e++) o[g][e] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < NF; j++) l_lane[j] = 0.f;

    int consumed = 0;
    for (int i = 0; i < n; i++) {
        const int s = i % C::STAGES;
        const bool got = mbar_wait(&full[s], (i / C::STAGES) & 1);
        if (!__syncthreads_and(got)) { if (threadIdx.x == 0) s_abort = 1; break; }
        consumed = i + 1;
        const uint8_t* ks = smem + s * C::STAGE_BYTES;
        const uint8_t* vs = ks + C::PAGE_BYTES;
        const int row0 = (pg_beg + i) * PAGE + warp * KPW;           // first row of this warp's keys

        // ---- partial dot products: vals[pass * G + g] over this lane's 8 dims
        float vals[N];
#pragma unroll
        for (int p = 0; p < NP; p++) {
            const int kk = warp * KPW + p * KP + kg;
            float kf[8];
            bf16x8_to_f32(*(const uint4*)(ks + (size_t)kk * HD * 2 + sub * 16), kf);
#pragma unroll
            for (int g = 0; g < G; g++) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < 8; e++) d = fmaf(q[g][e], kf[e], d);
                vals[p * G + g] = d;
            }
        }
        // ---- butterfly over the LPK lanes of a key: halves the values a lane holds at each step
        {
            int cnt = N;
#pragma unroll
            for (int off = LPK / 2; off >= 1; off >>= 1) {
                if (cnt > 1) {
                    cnt >>= 1;
                    const bool upper = (lane & off) != 0;
#pragma unroll
                    for (int j = 0; j < N / 2; j++) {
                        if (j < cnt) {
                            const float send = upper ? vals[j] : vals[j + cnt];
                            const float keep = upper ? vals[j + cnt] : vals[j];
                            vals[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                        }
                    }
                } else {
                    vals[0] += __shfl_xor_sync(0xffffffffu, vals[0], off);
                }
            }
        }
        // lane now holds NF scores: original index idx_j = (N > LPK) ? sub * NF + j : sub / SPREAD
        float sc[NF];
        int gh[NF];
        float pmax[G];
#pragma unroll
        for (int g = 0; g < G; g++) pmax[g] = -INFINITY;
#pragma unroll
        for (int j = 0; j < NF; j++) {
            const int idx = (N > LPK) ? sub * NF + j : sub / SPREAD;
            const int p = idx / G, g = idx % G;
            gh[j] = g;
            const int R = row0 + p * KP + kg;                       // row of this score's key
            bool valid;
            if (a.ring_rows > 0) {
                valid = R < min(len, a.ring_rows);
                if (valid) { const int pos = R + a.ring_rows * ((len - 1 - R) / a.ring_rows); valid = pos >= lo; }
            } else {
                valid = R >= lo && R < len;
            }
            float v = vals[j];
            if (a.cap > 0.f) v = softcap_f(v, a.cap);
            sc[j] = valid ? v : -INFINITY;
#pragma unroll
            for (int gg = 0; gg < G; gg++) if (gg == g) pmax[gg] = fmaxf(pmax[gg], sc[j]);
        }
#pragma unroll
        for (int g = 0; g < G; g++) pmax[g] = warp_max(pmax[g]);
        // ---- running softmax: one correction per page
        float corr[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float mn = fmaxf(m[g], pmax[g]);
            corr[g] = (mn == -INFINITY || m[g] == -INFINITY) ? 0.f : __expf(m[g] - mn);
            m[g] = mn;
#pragma unroll
            for (int e = 0; e < 8; e++) o[g][e] *= corr[g];
        }
        float pr[NF];
#pragma unroll
        for (int j = 0; j < NF; j++) {
            float mg = -INFINITY, cg = 0.f;
#pragma unroll
            for (int g = 0; g < G; g++) if (g == gh[j]) { mg = m[g]; cg = corr[g]; }
            pr[j] = (sc[j] == -INFINITY) ? 0.f : __expf(sc[j] - mg);
            l_lane[j] = l_lane[j] * cg + ((lane % SPREAD) == 0 ? pr[j] : 0.f);   // count each score once
        }
        // ---- o += p * v: fetch each (pass, head) probability from the lane that holds it
#pragma unroll
        for (int p = 0; p < NP; p++) {
            const int kk = warp * KPW + p * KP + kg;
            float pv[G];
            bool any = false;
#pragma unroll
            for (int g = 0; g < G; g++) {
                const int idx = p * G + g;
                const int src_sub = (N > LPK) ? idx / NF : idx * SPREAD;
                float val = 0.f;
#pragma unroll
                for (int j = 0; j < NF; j++) {
                    const float t = __shfl_sync(0xffffffffu, pr[j], kg * LPK + src_sub);
                    if ((N > LPK ? idx % NF : 0) == j) val = t;
                }
                pv[g] = val;
                any |= val != 0.f;
            }
            if (any) {                                              // rows that are not keys are never read
                float vf[8];
                bf16x8_to_f32(*(const uint4*)(vs + (size_t)kk * HD * 2 + sub * 16), vf);
#pragma unroll
                for (int g = 0; g < G; g++)
                    if (pv[g] != 0.f) {
#pragma unroll
                        for (int e = 0; e < 8; e++) o[g][e] = fmaf(pv[g], vf[e], o[g][e]);
                    }
            }
        }
        __syncthreads();                                            // everyone is done with stage s
        if (threadIdx.x == 0 && i + C::STAGES < n) issue(i + C::STAGES);
    }

    if (s_abort) {
        // a wait ran out: record it, and let copies that were issued land before the CTA ends
        if (threadIdx.x == 0) {
            atomicExch(&g_attn_error, 1);
            const int issued = min(n, consumed + C::STAGES);
            for (int i = consumed; i < issued; i++) mbar_wait(&full[i % C::STAGES], (i / C::STAGES) & 1);
        }
        __syncthreads();
        return;
    }

    // ---- fold the key groups of a warp, then the warps
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1)
#pragma unroll
        for (int g = 0; g < G; g++)
#pragma unroll
            for (int e = 0; e < 8; e++) o[g][e] += __shfl_xor_sync(0xffffffffu, o[g][e], off);
    float lsum[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < NF; j++) if ((((N > LPK) ? sub * NF + j : sub / SPREAD) % G) == g) t += l_lane[j];
        lsum[g] = warp_sum(t);
    }
    __syncthreads();                                                // the stages are free: reuse them
    float* red = (float*)smem;                                      // [NWARP][G][HD + 2]
    if (kg == 0) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            float* r = red + ((size_t)warp * G + g) * (HD + 2);
#pragma unroll
            for (int e = 0; e < 8; e++) r[sub * 8 + e] = o[g][e];
            if (sub == 0) { r[HD] = m[g]; r[HD + 1] = lsum[g]; }
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < G * HD; t += blockDim.x) {
        const int g = t / HD, d = t % HD;
        float M = -INFINITY;
        for (int w = 0; w < NWARP; w++) M = fmaxf(M, red[((size_t)w * G + g) * (HD + 2) + HD]);
        float L = 0.f, acc = 0.f;
        for (int w = 0; w < NWARP; w++) {
            const float* r = red + ((size_t)w * G + g) * (HD + 2);
            if (r[HD] != -INFINITY) { const float f = __expf(r[HD] - M); L += r[HD + 1] * f; acc += r[d] * f; }
        }
        const int h = kvh * G + g;
        if (a.n_splits == 1) {
            ((bf16*)a.out)[((size_t)b * a.n_heads + h) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            float* p = a.partial + (((size_t)b * a.n_heads + h) * a.n_splits + split) * (HD + 2);
            p[d] = acc;
            if (d == 0) { p[HD] = M; p[HD + 1] = L; }
        }
    }
}

// ---------------------------------------------------------------------------
// Tensor-core variant: a page's 64 keys are the rows of the MMA tiles, the group's query heads
// (up to 8) their 8 columns.
//
//   S^T = K Q^T   [64 keys x 8 heads]:  A = K rows as they lie in the page, B = Q held in registers
//   O^T = V^T P^T [head_dim x 8 heads]: A = V read through ldmatrix.trans, B = P^T built in registers
//
// as mma.sync m16n8k16 (bfloat16 operands, 32-bit accumulators).  With keys on the 16-row side no
// MMA row is wasted on padding, so a page costs head_dim/2 MMAs and as many ldmatrix for the whole
// CTA instead of some 5,000 scalar instructions, and the kernel's time is the time of its page
// copies.  A page arrives as head_dim/64 tiled TMA copies of 64 keys x 64 dims with the 128-byte
// swizzle (8 KB each), the layout in which every ldmatrix is conflict-free.
//
// The nine warps of a CTA have three roles and meet only through mbarriers (every wait bounded):
//   warps 0..3  scores: warp w multiplies the page's keys 16w..16w+15 with all of head_dim (four chains of
//               MMAs), applies scale, cap and the validity mask on the accumulators and leaves the scores and
//               their maximum per head in shared memory (two pages' worth, so that it may run a page ahead);
//   warps 4..7  outputs: each owns head_dim/4 dims of O^T: it reads the four maxima and the scores of the
//               page, updates the running maximum and sum (identically in all four warps), builds P^T in
//               registers and multiplies its slice of V^T with it;
//   warp 8      copies: one lane refills a stage as soon as all eight computing warps have let go of it, so the
//               page-table lookup and the copy instructions are on nobody's critical path.
// A page's dependent chain (wait, ldmatrix, MMAs, cap, maximum / exponentials, MMAs) is thus cut in two halves
// that overlap across pages; with one CTA-wide barrier per phase the same work took 1.37 us a page on an idle
// GPU, as much as the page's copy takes when all SMs stream.  Rows of a page that are not keys of the sequence
// get -inf scores, and their V rows are zeroed in shared memory before use (0 * NaN would still poison O).
//
// Before griddepcontrol.wait the kernel already fetches pages that this step does not write (all
// but the one that takes the new token): they were complete before the step began.
//
// Splits write (max, sum, O) partials; the CTA that finishes last for a (sequence, kv head), found
// with a ticket counter, folds them in split order, so the sum does not depend on which CTA that is
// (split partition: all eight computing warps fold; stream partition: the output warps, between two runs).
// ---------------------------------------------------------------------------
#define TW 8                                       // warps that compute: 0..3 the scores, 4..7 the outputs
#define NTHREADS ((TW + 1) * 32)                   // and one warp that issues the page copies
#define SROW 72                                    // floats between heads in the score arrays (64 keys + 8: no bank conflicts)
template <int HD, bool STREAM> struct MCfg {
    static constexpr int BOXES = HD / 64;                            // 64-dim column boxes per page
    static constexpr int BOX_BYTES = PAGE * 128;                     // 64 keys x 128 bytes, swizzled
    static constexpr int TILE_BYTES = BOXES * BOX_BYTES;             // one page of K (or V)
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    // One CTA an SM with the whole shared memory as stages; but the stream partition at heads narrower than 256 takes
    // half, so that two CTAs share an SM: a page of narrow heads is copied faster than its chain of dependent steps
    // runs through the two warp groups, and a second CTA's pages fill that time (27B shape, batch 64: 0.63 -> 0.77 of
    // the memory's speed).  The split partition serves small batches, where one CTA with six stages was faster.
    static constexpr int CTAS_PER_SM = (STREAM && HD <= 128) ? 2 : 1;
    static constexpr int STAGES_RAW = ((192 / CTAS_PER_SM) * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
    static constexpr int KS = HD / 16;                               // k-steps of S^T = K Q^T
    static constexpr int MT_W = HD / 64;                             // 16-dim tiles of O^T per output warp (head_dim / 4 dims)
    static constexpr int SCORE_FLOATS = 2 * 8 * SROW + 2 * 8 * 4;    // two pages' scores, and their maxima per score warp
    static constexpr int SMEM = STAGES * STAGE_BYTES + SCORE_FLOATS * 4 + 192 /* barriers */ + (1024 + 4) * 4 /* stream: page prefix */
                                + 8 * HD * 2 /* rotated queries */ + 10 * HD * 4 /* this step's q, k, v, summed */
                                + 32 /* fold job, abort flag */ + 1024 /* alignment */;
};
// byte offset of (key row r, 16-byte chunk c of the head dim) inside a swizzled page
__device__ __forceinline__ int sw_off(int r, int c) {
    return (c >> 3) * (PAGE * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// cap * tanh(x / cap) as cap * (1 - 2 / (e^(2x/cap) + 1)) with the fast exponential and division: the absolute
// error stays near cap * 2^-22, far below what rounding the probabilities to bfloat16 costs, at a tenth of the
// instructions of tanhf.  Large |x| saturate to +-cap without overflow trouble (e^y = inf gives 1, e^y = 0 gives -1).
__device__ __forceinline__ float softcap_fast(float x, float cap, float inv_cap) {
    const float e = __expf(2.f * x * inv_cap);
    return cap * (1.f - __fdividef(2.f, e + 1.f));
}

// How a launch's pages are dealt out to CTAs.
//   split:  grid (sequence, kv head, piece); a sequence's pages are cut into n_splits equal pieces
//           (the caller picks n_splits from the longest sequence).
//   stream: grid (CTAs); all pages of the launch, ordered by (sequence, kv head, page), are cut into
//           gridDim.x equal runs, wherever the sequences end.  Every SM gets the same number of pages
//           whatever the batch and the lengths are, and a CTA's copy pipeline never drains between
//           sequences.  A run that covers only part of a (sequence, kv head) leaves a partial: in the
//           CTA's slot 1 if it begins the pair, in slot 0 if it continues one.
#define STREAM_MAX_BATCH 1024
#define HOT_RUNS_MAX ((2 * 8 * SROW - 1) / 2)        // runs of one CTA that hold a new token's page: their list lies in the scores' place

// Walks pages in (sequence, kv head, page) order.  The same code runs in every thread (consumer side)
// and, ahead of it, in the thread that issues the copies.
struct PageCursor {
    int b, kvh, pg;            // sequence, kv head, page within the pair (0 = first page that holds keys)
    int np, first_page, hot;   // of sequence b: pages with keys, first of them (table index), the page this step writes
    int left;                  // pages still to visit
};

template <int HD, bool STREAM>
__global__ void __launch_bounds__(NTHREADS, MCfg<HD, STREAM>::CTAS_PER_SM)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, DecodeArgs a,
                       int batch) {
    pdl_launch_dependents();
    using C = MCfg<HD, STREAM>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* sf = (float*)(smem + C::STAGES * C::STAGE_BYTES);         // [page parity][8 heads][SROW] scores: scaled, capped, masked
    float* pm = sf + 2 * 8 * SROW;                                   // [page parity][8 heads][4] their maxima per score warp
    uint64_t* full = (uint64_t*)(pm + 2 * 8 * 4);                    // [STAGES] a page has landed
    uint64_t* empty = full + C::STAGES;                              // [STAGES] all eight warps are done with it
    uint64_t* s_full = empty + C::STAGES;                            // [2] the four score warps have written a page's scores
    uint64_t* s_empty = s_full + 2;                                  // [2] the four output warps have read them
    uint64_t* grp = s_empty + 2;                                     // [3] meeting points of the score warps, of the output warps, of all eight
    int* pref = (int*)(full + 24);                                   // stream: [batch + 1] pages before each sequence
    bf16* q_s = (bf16*)(pref + 1024 + 4);                            // [8 heads][HD] this run's queries, rotated (fused rotation)
    float* fold_s = (float*)(q_s + 8 * HD);                          // [G heads of q, then k, then v][HD]: the partial sums added up
    // (no static shared memory: two CTAs of this kernel fill an SM's shared memory to the last kilobyte)
    int* misc = (int*)(fold_s + 10 * HD);
    int& s_last = misc[0];                          // split: this CTA folds the pair below
    int* s_job = misc + 1;                          // the pair to fold (sequence, kv head, parts)
    volatile int& s_abort = *(volatile int*)(misc + 4);
    if ((uint8_t*)(misc + 8) > smem_raw + C::SMEM) {                 // the block began less aligned than the budget assumes
        if (threadIdx.x == 0) atomicExch(&g_attn_error, 2);
        return;
    }

    const int G = a.n_heads / a.n_kv_heads;                         // 1..8 query heads on columns 0..G-1
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane >> 2, t = lane & 3;

    // geometry of a sequence: its pages that hold keys, in row space (positions, or ring rows)
    auto seq_pages = [&](int b, int& first_page, int& hot) -> int {
        const int len = a.len_after[b];
        const int lo = (a.window > 0 && len > a.window) ? len - a.window : 0;
        hot = ((a.ring_rows > 0) ? (len - 1) % a.ring_rows : (len - 1)) / PAGE;
        if (a.ring_rows > 0) { first_page = 0; return (min(len, a.ring_rows) + PAGE - 1) / PAGE; }
        first_page = lo / PAGE;
        return (len - 1) / PAGE - first_page + 1;
    };

    if (tid == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], TW); }
        for (int u = 0; u < 2; u++) { mbar_init(&s_full[u], TW / 2); mbar_init(&s_empty[u], TW / 2); mbar_init(&grp[u], TW / 2); }
        mbar_init(&grp[2], TW);
        s_abort = 0;
        s_last = 0;
        mbar_init_fence();
    }
    if (tid == 32) {                                // the tensor maps, ahead of the first copy that uses them
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_v) : "memory");
    }

    PageCursor cur;
    long long g_beg = 0, total = 0;                                  // stream: this CTA's first page, all pages
    int n_ctas = 1;                                                  // stream: CTAs that take part
    if (STREAM) {
        // pages before each sequence (one kv head's worth), by warp 0
        if (warp == 0) {
            int carry = 0;
            for (int base = 0; base < batch; base += 32) {
                int fp, hot;
                int v = (base + lane < batch) ? seq_pages(base + lane, fp, hot) : 0;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
                if (base + lane < batch) pref[base + lane + 1] = carry + v;
                carry += __shfl_sync(0xffffffffu, v, 31);
            }
            if (lane == 0) pref[0] = 0;
        }
        __syncthreads();
        total = (long long)pref[batch] * a.n_kv_heads;
        n_ctas = (int)min((long long)gridDim.x, total);             // no CTA without a page: the rest leave
        if ((int)blockIdx.x >= n_ctas) return;
        g_beg = (long long)blockIdx.x * total / n_ctas;
        const long long g_end = (long long)(blockIdx.x + 1) * total / n_ctas;
        cur.left = (int)(g_end - g_beg);
        int lo_b = 0, hi_b = batch - 1;                              // the last sequence that begins at or before g_beg
        while (lo_b < hi_b) {
            const int mid = (lo_b + hi_b + 1) >> 1;
            if ((long long)pref[mid] * a.n_kv_heads <= g_beg) lo_b = mid; else hi_b = mid - 1;
        }
        cur.b = lo_b;
        cur.np = seq_pages(cur.b, cur.first_page, cur.hot);
        const int within = (int)(g_beg - (long long)pref[cur.b] * a.n_kv_heads);
        cur.kvh = within / cur.np;
        cur.pg = within % cur.np;
    } else {
        __syncthreads();
        cur.b = blockIdx.x; cur.kvh = blockIdx.y;
        cur.np = seq_pages(cur.b, cur.first_page, cur.hot);
        const int per = (cur.np + a.n_splits - 1) / a.n_splits;
        cur.pg = min(cur.np, (int)blockIdx.z * per);
        cur.left = min(per, cur.np - cur.pg);
    }
    auto advance = [&](PageCursor& c) {
        c.left--;
        if (++c.pg == c.np && c.left > 0) {
            c.pg = 0;
            if (++c.kvh == a.n_kv_heads) { c.kvh = 0; c.b++; c.np = seq_pages(c.b, c.first_page, c.hot); }
        }
    };

    // one thread issues the copies of a page: head_dim/64 boxes of K and as many of V
    PageCursor ahead = cur;
    int issued = 0;                                                  // pages whose copies are under way (issuing thread)
    constexpr int ISSUER = TW * 32;                                  // lane 0 of the ninth warp
    auto issue = [&]() {
        const int s = issued % C::STAGES;
        const int page = a.page_table[(size_t)ahead.b * a.pt_stride + ahead.first_page + ahead.pg];
        const int row = (page * a.n_kv_heads + ahead.kvh) * PAGE;   // row of the pool seen as [rows, head_dim]
        uint8_t* dst = smem + s * C::STAGE_BYTES;
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
#pragma unroll
        for (int bx = 0; bx < C::BOXES; bx++) {
            tma_load_box(dst + bx * C::BOX_BYTES, &map_k, &full[s], bx * 64, row);
            tma_load_box(dst + C::TILE_BYTES + bx * C::BOX_BYTES, &map_v, &full[s], bx * 64, row);
        }
        issued++;
        advance(ahead);
    };
    // pages that this step does not write were complete before the step began: fetch them at once
    if (tid == ISSUER)
        while (ahead.left > 0 && issued < C::STAGES && ahead.first_page + ahead.pg != ahead.hot) issue();
    pdl_wait();                                     // the new token's cache rows and q come from earlier kernels

    // ---- fused rotation: this step's q, k, v come as partial sums of their product
    const bool fused = a.qkv_part != nullptr;
    const int half = (a.inv_freq != nullptr) ? (a.rotary_dim >> 1) : 0;      // rotated pairs per head
    const int per = HD - half;                                               // items of a head: rotated pairs, then dims beyond them
    const int k_off = a.n_heads * HD, v_off = (a.n_heads + a.n_kv_heads) * HD;
    // Adds up partial sums into fold_s: segment g (HD columns) is the piece of sequence seg_b(g)'s row that begins at
    // column seg_col(g).  Every partial sum that is needed is requested at once, four columns a thread and eight
    // splits each, and added in the splits' order: one wait for memory.  For the nthr threads t0 = 0 .. nthr - 1.
    auto bulk_sum = [&](int n_seg, auto seg_b, auto seg_col, int t0, int nthr) {
        const int n_cols = n_seg * HD;
        for (int c0 = t0; c0 < n_cols; c0 += 4 * nthr) {
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            const float* src[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int c = min(c0 + e * nthr, n_cols - 1), g = c / HD;
                src[e] = a.qkv_part + (size_t)seg_b(g) * a.qkv_row_stride + seg_col(g) + (c - g * HD);
            }
            for (int s0 = 0; s0 < a.qkv_splits; s0 += 8) {
                float t8[4][8];
#pragma unroll
                for (int e = 0; e < 4; e++)
#pragma unroll
                    for (int k = 0; k < 8; k++)
                        if (c0 + e * nthr < n_cols && s0 + k < a.qkv_splits) t8[e][k] = src[e][(size_t)(s0 + k) * a.qkv_split_stride];
#pragma unroll
                for (int e = 0; e < 4; e++)
#pragma unroll
                    for (int k = 0; k < 8; k++)
                        if (c0 + e * nthr < n_cols && s0 + k < a.qkv_splits) sum[e] = (s0 + k == 0) ? t8[e][k] : sum[e] + t8[e][k];
            }
#pragma unroll
            for (int e = 0; e < 4; e++) if (c0 + e * nthr < n_cols) fold_s[c0 + e * nthr] = sum[e];
        }
    };
    // a head (its 32-bit values at hsrc) rotated at `pos` and rounded: item x is a rotated pair or a dim beyond the rotary part
    auto rotate_from = [&](const float* hsrc, bf16* dst, int x, int pos) {
        if (x < half) {
            float sn, cs;
            sincosf((float)pos * a.inv_freq[x], &sn, &cs);
            const float x0 = hsrc[x], x1 = hsrc[x + half];
            dst[x] = __float2bfloat16_rn(x0 * cs - x1 * sn);
            dst[x + half] = __float2bfloat16_rn(x1 * cs + x0 * sn);
        } else {
            dst[x + half] = __float2bfloat16_rn(hsrc[x + half]);
        }
    };
    // where the new token's k and v rows of (sequence b, kv head kvh) lie in the pools
    auto new_row = [&](int b, int kvh) -> size_t {
        const int pos = a.len_after[b] - 1;
        const int r = (a.ring_rows > 0) ? pos % a.ring_rows : pos;
        const int page = a.page_table[(size_t)b * a.pt_stride + r / PAGE];
        return ((size_t)(page * a.n_kv_heads + kvh) * PAGE + (r % PAGE)) * HD;
    };
    // k (32-bit at ksrc) rotated and v (at vsrc) rounded into the new token's rows, by the nthr threads t0 = 0 .. nthr - 1
    auto append_kv = [&](int b, int kvh, const float* ksrc, const float* vsrc, int t0, int nthr) {
        const size_t off = new_row(b, kvh);
        bf16* kd = (bf16*)a.k_pool + off;
        bf16* vd = (bf16*)a.v_pool + off;
        const int pos = a.len_after[b] - 1;
        for (int x = t0; x < per + HD; x += nthr) {
            if (x < per) rotate_from(ksrc, kd, x, pos);
            else vd[x - per] = __float2bfloat16_rn(vsrc[x - per]);
        }
    };
    if (fused && !STREAM) {
        // Split: the CTA has one run.  It needs its G query heads; k and v too if its run holds the page of the new
        // token, which this CTA and no other reads.
        const int pos = a.len_after[cur.b] - 1;
        const int hot_rel = cur.hot - cur.first_page;
        const bool hot_here = cur.left > 0 && hot_rel >= cur.pg && hot_rel < cur.pg + cur.left;
        if (warp < TW)
            bulk_sum(G + (hot_here ? 2 : 0), [&](int) { return cur.b; },
                     [&](int g) { return g < G ? (cur.kvh * G + g) * HD : g == G ? k_off + cur.kvh * HD : v_off + cur.kvh * HD; },
                     tid, TW * 32);
        __syncthreads();
        if (warp < TW) {
            for (int x = tid; x < G * per; x += TW * 32) rotate_from(fold_s + (x / per) * HD, q_s + (x / per) * HD, x % per, pos);
            if (hot_here) {
                append_kv(cur.b, cur.kvh, fold_s + G * HD, fold_s + (G + 1) * HD, tid, TW * 32);
                // the rows were written by ordinary stores and are read by the copy engine next
                __threadfence();
                asm volatile("fence.proxy.async;" ::: "memory");
            }
        }
        __syncthreads();
    } else if (fused) {
        // Stream: the CTA has one run or several.  Those that hold the page of their sequence's new token (this CTA,
        // and no other, reads that page) get the token's k and v rows written first; the first run's query heads go
        // to shared memory.  In passes of up to ten heads' worth of partial sums (what fold_s holds): the first pass
        // takes the G query heads and as many (k, v) pairs as fit beside them, the later ones five pairs each.
        int* hot_runs = (int*)sf;                                   // [0] how many, then (sequence, kv head) each; scores come later
        if (tid == 0) {
            int n = 0;
            PageCursor w = cur;
            while (w.left > 0) {
                const int nrun = min(w.left, w.np - w.pg), hot_rel = w.hot - w.first_page;
                if (hot_rel >= w.pg && hot_rel < w.pg + nrun) {
                    if (n == HOT_RUNS_MAX) { atomicExch(&g_attn_error, 3); s_abort = 1; break; }      // (the host refuses such launches)
                    hot_runs[1 + 2 * n] = w.b; hot_runs[2 + 2 * n] = w.kvh; n++;
                }
                w.left -= nrun;
                w.pg += nrun;
                if (w.pg == w.np && w.left > 0) {
                    w.pg = 0;
                    if (++w.kvh == a.n_kv_heads) { w.kvh = 0; w.b++; w.np = seq_pages(w.b, w.first_page, w.hot); }
                }
            }
            hot_runs[0] = n;
        }
        __syncthreads();
        const int n_hot = hot_runs[0];
        const int q_b = cur.b, q_kvh = cur.kvh, q_pos = a.len_after[cur.b] - 1;
        int done = 0;                                               // hot runs written so far
        for (int pass = 0; pass == 0 || done < n_hot; pass++) {
            const int nq = pass == 0 ? G : 0;                       // query heads in this pass
            const int take = min(n_hot - done, (10 - nq) / 2);
            if (warp < TW)
                bulk_sum(nq + 2 * take,
                         [&](int g) { return g < nq ? q_b : hot_runs[1 + 2 * (done + (g - nq) / 2)]; },
                         [&](int g) {
                             if (g < nq) return (q_kvh * G + g) * HD;
                             const int kvh = hot_runs[2 + 2 * (done + (g - nq) / 2)];
                             return ((g - nq) & 1) ? v_off + kvh * HD : k_off + kvh * HD;
                         },
                         tid, TW * 32);
            __syncthreads();
            if (warp < TW) {
                for (int x = tid; x < nq * per; x += TW * 32) rotate_from(fold_s + (x / per) * HD, q_s + (x / per) * HD, x % per, q_pos);
                // a pair of warps (64 threads) takes a hot run; four runs at a time
                for (int r = warp / 2; r < take; r += TW / 2)
                    append_kv(hot_runs[1 + 2 * (done + r)], hot_runs[2 + 2 * (done + r)], fold_s + (nq + 2 * r) * HD,
                              fold_s + (nq + 2 * r + 1) * HD, tid & 63, 64);
            }
            done += take;
            __syncthreads();                                        // fold_s is free for the next pass; q_s is written
        }
        // the rows were written by ordinary stores and are read by the copy engine next
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");
        __syncthreads();
    }
    if (tid == ISSUER) {
        if (fused) asm volatile("fence.proxy.async;" ::: "memory");
        while (ahead.left > 0 && issued < C::STAGES) issue();
    }

    const float inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;
    const uint32_t smem_base = smem_u32(smem);

    // A warp that gives up (a bounded wait ran out) says so; the others notice at their next wait.
    auto wait_on = [&](uint64_t* bar, uint32_t parity) -> bool {
        if (s_abort) return false;
        if (mbar_wait(bar, parity)) return true;
        s_abort = 1;
        return false;
    };
    // the four warps of a role meet (a bounded barrier): every lane waits until all four have arrived
    auto meet = [&](int which, uint32_t& phase) -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(&grp[which]);
        const bool ok = wait_on(&grp[which], phase & 1);
        phase++;
        return ok;
    };
    // geometry of the run that the cursor stands on: which rows (in row space) are keys.  Without a ring, or
    // before the ring has wrapped: lo <= R < len.  Once it has wrapped (len >= ring_rows) every row holds a token;
    // too old are the ring_rows - window rows that follow the newest one, a single circular run from old_beg.
    int len = 0, lo = 0, n_old = 0, old_beg = 0;
    bool wrapped = false, no_invalid = false;
    auto set_geometry = [&](int b) {
        len = a.len_after[b];
        lo = (a.window > 0 && len > a.window) ? len - a.window : 0;
        wrapped = a.ring_rows > 0 && len >= a.ring_rows;
        const int newest = wrapped ? (len - 1) % a.ring_rows : 0;
        n_old = wrapped ? a.ring_rows - a.window : 0;
        old_beg = wrapped ? (newest + 1 == a.ring_rows ? 0 : newest + 1) : 0;
        no_invalid = wrapped && n_old == 0;                         // a full ring whose every row is in the window
    };
    auto is_key = [&](int R) -> bool {
        if (wrapped) {
            int d = R - old_beg;                                    // distance past the start of the old run
            if (d < 0) d += a.ring_rows;
            return d >= n_old;
        }
        return R >= lo && R < len;
    };
    auto page_all_keys = [&](int row0) -> bool {
        if (no_invalid) return true;
        bool ok = is_key(row0) && is_key(row0 + PAGE - 1);
        // in a ring the rows that are too old form one circular run; it may lie inside the page
        if (wrapped && ok) ok = !(old_beg > row0 && old_beg <= row0 + PAGE - 1);
        return ok;
    };
    auto next_run = [&](PageCursor& c, int n) {                     // the cursor moves past a run of n pages
        c.left -= n;
        c.pg += n;
        if (c.pg == c.np && c.left > 0) {
            c.pg = 0;
            if (++c.kvh == a.n_kv_heads) { c.kvh = 0; c.b++; c.np = seq_pages(c.b, c.first_page, c.hot); }
        }
    };

    if (warp == TW) {
        // ================= the copies: a stage is refilled when all eight warps have let go of it =================
        if (lane == 0) {
            bool ok = true;
            while (ahead.left > 0) {
                const int s = issued % C::STAGES;
                if (issued >= C::STAGES && !wait_on(&empty[s], ((issued / C::STAGES) - 1) & 1)) { ok = false; break; }
                issue();
            }
            if (!ok || s_abort) {
                // a wait ran out: record it, and let copies that were issued land before the CTA ends
                atomicExch(&g_attn_error, 1);
                for (int j = max(0, issued - C::STAGES); j < issued; j++) mbar_wait(&full[j % C::STAGES], (j / C::STAGES) & 1);
            }
        }
    } else if (warp < TW / 2) {
        // ================= scores: S^T = K Q^T of this warp's 16 keys, scaled, capped, masked =================
        const int mt = warp;
        uint32_t koff[C::KS];                                       // where this lane's ldmatrix rows lie inside a stage
#pragma unroll
        for (int ks = 0; ks < C::KS; ks++)
            koff[ks] = sw_off(mt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), ks * 2 + (lane >> 4));
        uint32_t meet_phase = 0;
        int i = 0;                                                  // pages done
        bool first_run = true;
        while (cur.left > 0) {
            const int b = cur.b, kvh = cur.kvh, seg_pg0 = cur.pg, seg_n = min(cur.left, cur.np - cur.pg);
            const int seg_first = cur.first_page;
            set_geometry(b);
            // B fragments of Q^T: b0 = Q[head quad][16 ks + 2t, +1], b1 = Q[head quad][16 ks + 8 + 2t, +1]; heads >= G zero
            const bf16* qp = (const bf16*)a.q + (size_t)b * a.q_stride + (size_t)(kvh * G + quad) * HD;
            if (fused) {
                // the pair's query heads, rotated, go through shared memory (the first run's are there already)
                if (!first_run) {
                    // the run's partial sums are requested at once and added up in fold_s (nothing else uses it now)
                    bulk_sum(G, [&](int) { return b; }, [&](int g) { return (kvh * G + g) * HD; }, tid, (TW / 2) * 32);
                    if (!meet(0, meet_phase)) break;                // the sums are there; nobody reads the run before's queries any more
                    for (int x = tid; x < G * per; x += (TW / 2) * 32)
                        rotate_from(fold_s + (x / per) * HD, q_s + (x / per) * HD, x % per, len - 1);
                    if (!meet(0, meet_phase)) break;
                }
                qp = q_s + quad * HD;
            }
            first_run = false;
            uint32_t qb[C::KS][2];
#pragma unroll
            for (int ks = 0; ks < C::KS; ks++) {
                qb[ks][0] = (quad < G) ? *(const uint32_t*)(qp + ks * 16 + 2 * t) : 0u;
                qb[ks][1] = (quad < G) ? *(const uint32_t*)(qp + ks * 16 + 8 + 2 * t) : 0u;
            }
            bool ok = true;
            for (int j = 0; j < seg_n; j++, i++) {
                const int s = i % C::STAGES, u = i & 1;
                if (!wait_on(&full[s], (i / C::STAGES) & 1) || !wait_on(&s_empty[u], ((i >> 1) & 1) ^ 1)) { ok = false; break; }
                const uint32_t stage = smem_base + s * C::STAGE_BYTES;
                const int row0 = (seg_first + seg_pg0 + j) * PAGE;
                const bool all_ok = page_all_keys(row0);
                float c[4][4];                                       // four chains: the MMAs of a chain wait for one another
#pragma unroll
                for (int x = 0; x < 4; x++) { c[x][0] = c[x][1] = c[x][2] = c[x][3] = 0.f; }
#pragma unroll
                for (int ks = 0; ks < C::KS; ks++) {
                    uint32_t a0, a1, a2, a3;
                    ldsm_x4(stage + koff[ks], a0, a1, a2, a3);
                    mma_16816(c[ks & 3], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
                }
                // the accumulators hold keys quad, quad + 8 for heads 2t, 2t + 1
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int h = 2 * t + (e & 1), key = mt * 16 + quad + (e >> 1) * 8;
                    float v = ((c[0][e] + c[1][e]) + (c[2][e] + c[3][e])) * a.scale;
                    if (a.cap > 0.f) v = softcap_fast(v, a.cap, inv_cap);
                    if (!(all_ok || is_key(row0 + key))) v = -INFINITY;
                    if (h < G) sf[(u * 8 + h) * SROW + key] = v;
                    mx[e & 1] = fmaxf(mx[e & 1], v);
                }
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {                  // over the warp's keys: lanes that differ in quad
                    mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
                    mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
                }
                if (quad == 0) { pm[(u * 8 + 2 * t) * 4 + mt] = mx[0]; pm[(u * 8 + 2 * t + 1) * 4 + mt] = mx[1]; }
                __syncwarp();
                if (lane == 0) { mbar_arrive(&s_full[u]); mbar_arrive(&empty[s]); }
            }
            if (!ok) break;
            next_run(cur, seg_n);
        }
    } else {
        // ================= outputs: running softmax, O^T += V^T P^T for head_dim / 4 dims of this warp =================
        const int ow = warp - TW / 2;
        const int d0 = ow * (HD / 4);
        uint32_t voff[C::MT_W][4];
#pragma unroll
        for (int m = 0; m < C::MT_W; m++)
#pragma unroll
            for (int ks = 0; ks < 4; ks++)
                voff[m][ks] = C::TILE_BYTES + sw_off(ks * 16 + (lane >> 4) * 8 + (lane & 7), (d0 + m * 16) / 8 + ((lane >> 3) & 1));
        uint32_t meet_phase = 0;
        int i = 0;
        bool once = !STREAM;                                        // (split only) an empty piece still reports "nothing here"
        while (cur.left > 0 || once) {
            once = false;
            const int b = cur.b, kvh = cur.kvh, seg_pg0 = cur.pg, seg_n = min(cur.left, cur.np - cur.pg), seg_np = cur.np;
            const int seg_first = cur.first_page;
            set_geometry(b);
            float o[C::MT_W][4], o2[C::MT_W][4];                    // accumulator rows are dims, columns heads 2t, 2t+1; two chains
#pragma unroll
            for (int m = 0; m < C::MT_W; m++) { o[m][0] = o[m][1] = o[m][2] = o[m][3] = 0.f; o2[m][0] = o2[m][1] = o2[m][2] = o2[m][3] = 0.f; }
            // running maximum of the heads this lane meets: `quad` (its P^T column) and 2t, 2t+1 (its O^T columns)
            float m_b = -INFINITY, m_c0 = -INFINITY, m_c1 = -INFINITY, l_b = 0.f;
            bool ok = true;
            for (int j = 0; j < seg_n; j++, i++) {
                const int s = i % C::STAGES, u = i & 1;
                if (!wait_on(&s_full[u], (i >> 1) & 1)) { ok = false; break; }
                // the page's maximum per head from the four score warps; the scores of this lane's 16 keys for head quad
                const float4 qb4 = *(const float4*)(pm + (u * 8 + quad) * 4);
                const float4 c04 = *(const float4*)(pm + (u * 8 + 2 * t) * 4), c14 = *(const float4*)(pm + (u * 8 + 2 * t + 1) * 4);
                float sc[4][4];
                {
                    const float* s0 = sf + (u * 8 + (quad < G ? quad : 0)) * SROW + 2 * t;
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        const float2 x = *(const float2*)(s0 + ks * 16), y = *(const float2*)(s0 + ks * 16 + 8);
                        sc[ks][0] = x.x; sc[ks][1] = x.y; sc[ks][2] = y.x; sc[ks][3] = y.y;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[u]);
                const float pb_max = quad < G ? fmaxf(fmaxf(qb4.x, qb4.y), fmaxf(qb4.z, qb4.w)) : -INFINITY;
                const float pc0 = 2 * t < G ? fmaxf(fmaxf(c04.x, c04.y), fmaxf(c04.z, c04.w)) : -INFINITY;
                const float pc1 = 2 * t + 1 < G ? fmaxf(fmaxf(c14.x, c14.y), fmaxf(c14.z, c14.w)) : -INFINITY;
                const float nb = fmaxf(m_b, pb_max), n0 = fmaxf(m_c0, pc0), n1 = fmaxf(m_c1, pc1);
                const float sb = (nb == -INFINITY) ? 0.f : nb;
                const float corr_b = (m_b == -INFINITY) ? 0.f : __expf(m_b - sb);
                const float corr0 = (m_c0 == -INFINITY) ? 0.f : __expf(m_c0 - ((n0 == -INFINITY) ? 0.f : n0));
                const float corr1 = (m_c1 == -INFINITY) ? 0.f : __expf(m_c1 - ((n1 == -INFINITY) ? 0.f : n1));
                m_b = nb; m_c0 = n0; m_c1 = n1;
                uint32_t pb[4][2];
                float ps = 0.f;
                if (quad < G) {
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        const float p0 = __expf(sc[ks][0] - sb), p1 = __expf(sc[ks][1] - sb), p2 = __expf(sc[ks][2] - sb), p3 = __expf(sc[ks][3] - sb);
                        ps += (p0 + p1) + (p2 + p3);
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
                        pb[ks][0] = *(uint32_t*)&h0; pb[ks][1] = *(uint32_t*)&h1;
                    }
                } else {
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) { pb[ks][0] = 0u; pb[ks][1] = 0u; }
                }
                l_b = l_b * corr_b + ps;
                // the page's values (the score warps have seen it land; so does this warp)
                if (!wait_on(&full[s], (i / C::STAGES) & 1)) { ok = false; break; }
                const uint32_t stage = smem_base + s * C::STAGE_BYTES;
                const int row0 = (seg_first + seg_pg0 + j) * PAGE;
                const bool all_ok = page_all_keys(row0);
                if (!all_ok) {
                    // rows of the page that are not keys: their probabilities are 0, but 0 * NaN would still poison O,
                    // so this warp zeroes them in the columns it reads
                    uint8_t* v_s = smem + s * C::STAGE_BYTES + C::TILE_BYTES;
                    for (int x = lane; x < PAGE * (HD / 32); x += 32) {
                        const int r = x / (HD / 32), cc = d0 / 8 + x % (HD / 32);
                        if (!is_key(row0 + r)) *(uint4*)(v_s + sw_off(r, cc)) = make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
#pragma unroll
                for (int m = 0; m < C::MT_W; m++) {
                    o[m][0] *= corr0; o[m][1] *= corr1; o[m][2] *= corr0; o[m][3] *= corr1;
                    o2[m][0] *= corr0; o2[m][1] *= corr1; o2[m][2] *= corr0; o2[m][3] *= corr1;
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        uint32_t a0, a1, a2, a3;
                        ldsm_x4_t(stage + voff[m][ks], a0, a1, a2, a3);
                        mma_16816((ks & 1) ? o2[m] : o[m], a0, a1, a2, a3, pb[ks][0], pb[ks][1]);
                    }
                }
                // rows zeroed by ordinary stores; the stage is refilled by the copy engine
                if (!all_ok) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
            next_run(cur, seg_n);

            // ---- the run is done.  The sums of the quad's four lanes are the head's sum (the same in every warp).
#pragma unroll
            for (int m = 0; m < C::MT_W; m++) { o[m][0] += o2[m][0]; o[m][1] += o2[m][1]; o[m][2] += o2[m][2]; o[m][3] += o2[m][3]; }
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
            const float L0 = __shfl_sync(0xffffffffu, l_b, 4 * (2 * t)), L1 = __shfl_sync(0xffffffffu, l_b, 4 * (2 * t + 1));
            const bool begins = seg_pg0 == 0, whole = STREAM ? (begins && seg_n == seg_np) : (a.n_splits == 1);
            // where the parts of this (sequence, kv head) lie, and how many there are
            int n_parts, my_part, c_first = 0;
            if (STREAM) {
                const long long g0 = (long long)pref[b] * a.n_kv_heads + (long long)kvh * seg_np;   // the pair's first page
                c_first = (int)(((g0 + 1) * n_ctas - 1) / total);   // the CTA whose run holds page g: floor(((g + 1) n - 1) / total)
                const int c_last = (int)(((g0 + seg_np) * n_ctas - 1) / total);
                n_parts = c_last - c_first + 1;
                my_part = blockIdx.x - c_first;
            } else {
                n_parts = a.n_splits;
                my_part = blockIdx.z;
            }
            auto part_of = [&](int k, int hg) -> float* {           // part k of head hg of this pair
                if (STREAM) return a.partial + ((size_t)((c_first + k) * 2 + (k == 0 ? 1 : 0)) * G + hg) * (HD + 2);
                return a.partial + (((size_t)b * a.n_heads + kvh * G + hg) * a.n_splits + k) * (HD + 2);
            };
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int hg = 2 * t + e;
                if (hg >= G) continue;
                const float L = e ? L1 : L0, M = e ? m_c1 : m_c0;
                if (whole) {
                    bf16* dst = (bf16*)a.out + ((size_t)b * a.n_heads + kvh * G + hg) * HD;
#pragma unroll
                    for (int m = 0; m < C::MT_W; m++) {
                        dst[d0 + m * 16 + quad] = __float2bfloat16_rn(o[m][e] / L);
                        dst[d0 + m * 16 + quad + 8] = __float2bfloat16_rn(o[m][2 + e] / L);
                    }
                } else {
                    float* dst = part_of(my_part, hg);
#pragma unroll
                    for (int m = 0; m < C::MT_W; m++) {
                        dst[d0 + m * 16 + quad] = o[m][e];
                        dst[d0 + m * 16 + quad + 8] = o[m][2 + e];
                    }
                    if (ow == 0 && quad == 0) { dst[HD] = M; dst[HD + 1] = L; }
                }
            }
            if (whole || a.tickets == nullptr) continue;

            // ---- the CTA that finishes the pair's last part folds the parts, in their order.  The parts were written by
            // all four output warps; their meeting orders them before the counting, which is a release (for this CTA's
            // part) and an acquire (for the others') at GPU scope.
            if (!meet(1, meet_phase)) break;
            if (ow == 0 && lane == 0) {
                int* ticket = a.tickets + (size_t)b * a.n_kv_heads + kvh;
                int old;
                asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(ticket) : "memory");
                s_last = (old == n_parts - 1);
                if (s_last) *ticket = 0;                            // left at zero for the next launch
                s_job[0] = b; s_job[1] = kvh; s_job[2] = n_parts;
            }
            if (!meet(1, meet_phase)) break;
            if (!STREAM) break;                                     // split: one run; all eight warps fold it together below
            if (s_last) {
                for (int x = tid - (TW / 2) * 32; x < G * HD; x += (TW / 2) * 32) {
                    const int hg = x / HD, d = x % HD;
                    // out = sum_k e^(m_k - M) o_k / sum_k e^(m_k - M) l_k in the parts' order, eight parts requested at a
                    // time; M is the running maximum, by which the sums so far are rescaled
                    float M = -INFINITY, L = 0.f, acc = 0.f;
                    for (int k0 = 0; k0 < n_parts; k0 += 8) {
                        float ms[8], ls[8], os[8];
#pragma unroll
                        for (int k = 0; k < 8; k++)
                            if (k0 + k < n_parts) {
                                const float* pk = part_of(k0 + k, hg);
                                ms[k] = __ldcg(pk + HD); ls[k] = __ldcg(pk + HD + 1); os[k] = __ldcg(pk + d);
                            }
                        float Mn = M;
#pragma unroll
                        for (int k = 0; k < 8; k++) if (k0 + k < n_parts) Mn = fmaxf(Mn, ms[k]);
                        if (Mn == -INFINITY) continue;
                        const float r = (M == -INFINITY) ? 0.f : __expf(M - Mn);
                        L *= r; acc *= r; M = Mn;
#pragma unroll
                        for (int k = 0; k < 8; k++)
                            if (k0 + k < n_parts && ms[k] != -INFINITY) { const float f = __expf(ms[k] - M); L += ls[k] * f; acc += os[k] * f; }
                    }
                    ((bf16*)a.out)[((size_t)b * a.n_heads + kvh * G + hg) * HD + d] = __float2bfloat16_rn(acc / L);
                }
            }
            if (!meet(1, meet_phase)) break;                        // s_last is rewritten by the next run
        }
    }
    if (!STREAM && warp < TW && a.n_splits > 1 && a.tickets != nullptr) {
        // split: the CTA had one run.  If it was the pair's last part, all eight warps fold the parts:
        // out = sum_k w_k o_k with w_k = e^(m_k - M) / sum_j e^(m_j - M) l_j and M the largest m.  The parts' outputs are
        // requested first (two outputs a thread, 32 parts each), the weights are made meanwhile by one warp a head from
        // the parts' m and l, and the sum runs in the parts' order: one wait for memory, whatever else the GPU is doing.
        __syncwarp();
        if (lane == 0) mbar_arrive(&grp[2]);
        if (!wait_on(&grp[2], 0) || !s_last) return;
        const int b = s_job[0], kvh = s_job[1], n_parts = s_job[2];
        float* wts = sf;                                            // [8 heads][64 parts] (the scores' place; the run is over)
        constexpr int FK = 32;
        const float* p0 = a.partial + ((size_t)b * a.n_heads + kvh * G) * a.n_splits * (HD + 2);
        const size_t head_stride = (size_t)a.n_splits * (HD + 2);
        bool have_weights = false;
        for (int x0 = tid; x0 < G * HD || !have_weights; x0 += 2 * TW * 32) {
            float acc[2] = {0.f, 0.f};
            for (int k0 = 0; k0 < n_parts; k0 += FK) {
                float os[2][FK];
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int x = x0 + e * TW * 32;
                    if (x < G * HD) {
                        const float* px = p0 + (x / HD) * head_stride + (x % HD);
#pragma unroll
                        for (int k = 0; k < FK; k++) if (k0 + k < n_parts) os[e][k] = __ldcg(px + (size_t)(k0 + k) * (HD + 2));
                    }
                }
                if (!have_weights) {
                    if (warp < G) {
                        const float* ph = p0 + warp * head_stride;
                        float m[2], l[2], M = -INFINITY;
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const int k = lane + 32 * e;
                            m[e] = k < n_parts ? __ldcg(ph + (size_t)k * (HD + 2) + HD) : -INFINITY;
                            l[e] = k < n_parts ? __ldcg(ph + (size_t)k * (HD + 2) + HD + 1) : 0.f;
                            M = fmaxf(M, m[e]);
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
                        float f[2], L = 0.f;
#pragma unroll
                        for (int e = 0; e < 2; e++) { f[e] = (m[e] == -INFINITY) ? 0.f : __expf(m[e] - M); L += f[e] * l[e]; }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
                        const float inv = 1.f / L;
#pragma unroll
                        for (int e = 0; e < 2; e++) wts[warp * 64 + lane + 32 * e] = f[e] * inv;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&grp[2]);
                    if (!wait_on(&grp[2], 1)) return;
                    have_weights = true;
                }
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int x = x0 + e * TW * 32;
                    if (x < G * HD) {
                        const float* w = wts + (x / HD) * 64 + k0;
#pragma unroll
                        for (int k = 0; k < FK; k++) if (k0 + k < n_parts) acc[e] = fmaf(w[k], os[e][k], acc[e]);
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int x = x0 + e * TW * 32;
                if (x < G * HD) ((bf16*)a.out)[((size_t)b * a.n_heads + kvh * G + x / HD) * HD + x % HD] = __float2bfloat16_rn(acc[e]);
            }
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}
// A cache pool seen as a matrix [rows = pages * kv_heads * 64, head_dim]; box = 64 rows x 64 dims.
static int pool_map(CUtensorMap* m, const void* pool, long long rows, int hd) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return tb_refuse("attn_decode: the driver does not provide cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, PAGE};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)pool, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return tb_refuse("attn_decode: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

template <int HD, bool STREAM>
static int launch_mma(const DecodeArgs& a, int batch, int n_ctas, cudaStream_t stream) {
    using C = MCfg<HD, STREAM>;
    static bool attr_set = false;
    auto kern = attn_decode_mma_kernel<HD, STREAM>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    // the map's row count only bounds the copy engine's address check; pages come from the table
    const long long pool_rows = 0x7fffff00LL;
    CUtensorMap mk, mv;
    if (pool_map(&mk, a.k_pool, pool_rows, HD) || pool_map(&mv, a.v_pool, pool_rows, HD)) return -1;
    dim3 grid(batch, a.n_kv_heads, a.n_splits);
    if (STREAM) grid = dim3(n_ctas);
    tb_launch(kern, dim3(grid), dim3(NTHREADS), C::SMEM, stream, mk, mv, a, batch);
    return tb_launch_status();
}

// out[b,h,:] = sum_s e^(m_s - M) o_s / sum_s e^(m_s - M) l_s, splits in ascending order.
__global__ void attn_combine_kernel(const float* __restrict__ partial, bf16* __restrict__ out, int n_splits, int hd) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t bh = blockIdx.x;
    const float* p = partial + bh * n_splits * (hd + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, p[(size_t)s * (hd + 2) + hd]);
    float L = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = p[(size_t)s * (hd + 2) + hd];
        if (ms != -INFINITY) L += p[(size_t)s * (hd + 2) + hd + 1] * __expf(ms - M);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float ms = p[(size_t)s * (hd + 2) + hd];
            if (ms != -INFINITY) o += p[(size_t)s * (hd + 2) + d] * __expf(ms - M);
        }
        out[bh * hd + d] = __float2bfloat16_rn(o / L);
    }
}

template <int HD, int G>
static int launch(const DecodeArgs& a, int batch, cudaStream_t stream) {
    using C = DCfg<HD>;
    static bool attr_set = false;
    auto kern = attn_decode_kernel<HD, G>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    dim3 grid(batch, a.n_kv_heads, a.n_splits);
    tb_launch(kern, dim3(grid), dim3(C::NWARP * 32), C::SMEM, stream, a);
    return tb_launch_status();
}

extern "C" int tb_attn_decode_takes(int dtype, int n_heads, int n_kv_heads, int hd) {
    if (dtype != TB_BF16 || n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    const int g = n_heads / n_kv_heads;
    if (!(hd == 32 || hd == 64 || hd == 128 || hd == 256)) return 0;
    if (g < 1 || g > 8) return 0;
    if (hd == 32 && !(g == 1 || g == 2 || g == 4 || g == 8)) return 0;
    return 1;
}

static int run_decode(const DecodeArgs* args, int dtype, int batch, bool tensor_cores, cudaStream_t stream);

static int check_rotation(const DecodeArgs& a) {
    if (a.qkv_splits < 1 || a.qkv_row_stride < (long long)(a.n_heads + 2 * a.n_kv_heads) * a.hd)
        return tb_refuse("attn_decode: the q/k/v partial sums need at least one split and rows of (n_heads + 2 n_kv_heads) * head_dim");
    if (a.inv_freq != nullptr && (a.rotary_dim <= 0 || (a.rotary_dim & 1) || a.rotary_dim > a.hd))
        return tb_refuse("attn_decode: rotary_dim=%d must be even and within head_dim=%d", a.rotary_dim, a.hd);
    return 0;
}

// The product path: tensor-core variant.
extern "C" int tb_attn_decode(const DecodeArgs* args, int dtype, int batch, cudaStream_t stream) {
    return run_decode(args, dtype, batch, true, stream);
}
// The scalar variant (one lane group per key), kept for comparison in tests and measurements.
extern "C" int tb_attn_decode_lanes(const DecodeArgs* args, int dtype, int batch, cudaStream_t stream) {
    return run_decode(args, dtype, batch, false, stream);
}

static int run_decode(const DecodeArgs* args, int dtype, int batch, bool tensor_cores, cudaStream_t stream) {
    if (batch <= 0) return 0;
    DecodeArgs a = *args;
    if (!tb_attn_decode_takes(dtype, a.n_heads, a.n_kv_heads, a.hd))
        return tb_refuse("attn_decode: takes bfloat16, head_dim 32/64/128/256 and 1 to 8 heads per kv head "
                         "(got dtype %d, %d heads, %d kv heads, head_dim %d)", dtype, a.n_heads, a.n_kv_heads, a.hd);
    if (a.page_rows != PAGE) return tb_refuse("attn_decode: pages of %d rows, this kernel is built for %d", a.page_rows, PAGE);
    if (a.n_splits < 1 || a.n_splits > 65535 || a.n_kv_heads > 65535) return tb_refuse("attn_decode: n_splits=%d", a.n_splits);
    if (a.n_splits > 1 && a.partial == nullptr) return tb_refuse("attn_decode: splits need scratch");
    if (a.ring_rows > 0 && (a.ring_rows % PAGE || a.window <= 0 || a.window > a.ring_rows))
        return tb_refuse("attn_decode: a ring of %d rows cannot hold a window of %d", a.ring_rows, a.window);
    if (((uintptr_t)a.q & 15) || (a.q_stride % 8) || ((uintptr_t)a.k_pool & 15) || ((uintptr_t)a.v_pool & 15))
        return tb_refuse("attn_decode: q rows and the pools must be 16-byte aligned");
    const int g = a.n_heads / a.n_kv_heads;
    int st = -1;
    if (a.hd < 64) tensor_cores = false;            // a 64-byte row has no 128-byte swizzled box
    if (a.n_splits > 64) a.tickets = nullptr;       // the fold inside the kernel holds the weights of 64 pieces: more go to the fold launch
    if (a.qkv_part != nullptr) {
        if (!tensor_cores) return tb_refuse("attn_decode: only the tensor-core kernel (head_dim >= 64) rotates by itself");
        if (int r = check_rotation(a)) return r;
    } else if (a.q == nullptr) return tb_refuse("attn_decode: q is missing");
    if (tensor_cores) {
        switch (a.hd) {
        case 64: st = launch_mma<64, false>(a, batch, 0, stream); break;
        case 128: st = launch_mma<128, false>(a, batch, 0, stream); break;
        default: st = launch_mma<256, false>(a, batch, 0, stream); break;
        }
    } else {
    if (!(g == 1 || g == 2 || g == 4 || g == 8))
        return tb_refuse("attn_decode_lanes: %d heads per kv head (takes 1, 2, 4 or 8)", g);
#define GO(HD_)                                                          \
    switch (g) {                                                         \
    case 1: st = launch<HD_, 1>(a, batch, stream); break;                \
    case 2: st = launch<HD_, 2>(a, batch, stream); break;                \
    case 4: st = launch<HD_, 4>(a, batch, stream); break;                \
    default: st = launch<HD_, 8>(a, batch, stream); break;               \
    }
    switch (a.hd) {
    case 32: GO(32); break;
    case 64: GO(64); break;
    case 128: GO(128); break;
    default: GO(256); break;
    }
#undef GO
    }
    if (st) return st;
    if (a.n_splits > 1 && !(tensor_cores && a.tickets != nullptr)) {
        tb_launch(attn_combine_kernel, dim3((unsigned)batch * a.n_heads), dim3(128), 0, stream, a.partial, (bf16*)a.out, a.n_splits, a.hd);
        st = tb_launch_status();
    }
    return st;
}

// The tensor-core kernel with the launch's pages dealt out evenly to `n_ctas` CTAs (see "stream" above): no
// piece count to choose, every SM equally loaded whatever the lengths are.  `args->n_splits` is ignored;
// `args->partial` must hold tb_attn_decode_stream_scratch_floats() floats and `args->tickets` batch * n_kv_heads
// zeroed counters, which the launch leaves at zero.
// CTAs of the tensor-core kernel that fit an SM together (the stream partition's shared memory and registers are
// budgeted for two at heads narrower than 256; one everywhere else); -1 on error.
template <int HD, bool STREAM> static int mma_occupancy() {
    using C = MCfg<HD, STREAM>;
    int n = 0;
    cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<HD, STREAM>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_mma_kernel<HD, STREAM>, NTHREADS, C::SMEM);
    return e == cudaSuccess ? n : -1;
}
extern "C" int tb_attn_decode_occupancy(int hd, int stream_partition) {
    switch (hd) {
    case 64: return stream_partition ? mma_occupancy<64, true>() : mma_occupancy<64, false>();
    case 128: return stream_partition ? mma_occupancy<128, true>() : mma_occupancy<128, false>();
    case 256: return stream_partition ? mma_occupancy<256, true>() : mma_occupancy<256, false>();
    default: return -1;
    }
}

// How many CTAs a stream launch should use on a GPU of `sms` SMs (two an SM for heads narrower than 256).
extern "C" int tb_attn_decode_stream_ctas(int sms, int hd) { return sms * (hd <= 128 ? 2 : 1); }
extern "C" long long tb_attn_decode_stream_scratch_floats(int n_ctas, int n_heads, int n_kv_heads, int hd) {
    return (long long)n_ctas * 2 * (n_heads / (n_kv_heads > 0 ? n_kv_heads : 1)) * (hd + 2);
}
extern "C" int tb_attn_decode_stream(const DecodeArgs* args, int dtype, int batch, int n_ctas, cudaStream_t stream) {
    if (batch <= 0) return 0;
    DecodeArgs a = *args;
    if (!tb_attn_decode_takes(dtype, a.n_heads, a.n_kv_heads, a.hd) || a.hd < 64)
        return tb_refuse("attn_decode_stream: takes bfloat16, head_dim 64/128/256 and 1 to 8 heads per kv head "
                         "(got dtype %d, %d heads, %d kv heads, head_dim %d)", dtype, a.n_heads, a.n_kv_heads, a.hd);
    if (a.page_rows != PAGE) return tb_refuse("attn_decode: pages of %d rows, this kernel is built for %d", a.page_rows, PAGE);
    if (batch > STREAM_MAX_BATCH) return tb_refuse("attn_decode_stream: batch %d, takes up to %d", batch, STREAM_MAX_BATCH);
    if (n_ctas < 1 || n_ctas > 65535) return tb_refuse("attn_decode_stream: n_ctas=%d", n_ctas);
    // a CTA's runs are at most its share of the (sequence, kv head) pairs and one more
    if (a.qkv_part != nullptr && ((long long)batch * a.n_kv_heads + n_ctas - 1) / n_ctas + 1 > HOT_RUNS_MAX)
        return tb_refuse("attn_decode_stream: %d sequences x %d kv heads on %d CTAs are more runs per CTA than the fused rotation takes (%d)",
                         batch, a.n_kv_heads, n_ctas, HOT_RUNS_MAX);
    if (a.partial == nullptr || a.tickets == nullptr) return tb_refuse("attn_decode_stream: needs scratch and ticket counters");
    if (a.qkv_part != nullptr) { if (int r = check_rotation(a)) return r; }
    else if (a.q == nullptr) return tb_refuse("attn_decode_stream: q is missing");
    if (a.ring_rows > 0 && (a.ring_rows % PAGE || a.window <= 0 || a.window > a.ring_rows))
        return tb_refuse("attn_decode: a ring of %d rows cannot hold a window of %d", a.ring_rows, a.window);
    if (((uintptr_t)a.q & 15) || (a.q_stride % 8) || ((uintptr_t)a.k_pool & 15) || ((uintptr_t)a.v_pool & 15))
        return tb_refuse("attn_decode: q rows and the pools must be 16-byte aligned");
    a.n_splits = 0;
    switch (a.hd) {
    case 64: return launch_mma<64, true>(a, batch, n_ctas, stream);
    case 128: return launch_mma<128, true>(a, batch, n_ctas, stream);
    default: return launch_mma<256, true>(a, batch, n_ctas, stream);
    }
}

// ---------------------------------------------------------------------------
// An entry point that allocates nothing (declared in attention_decode_noalloc.h; it has no
// counterpart in the reference).
//
// tb_attn_decode wants its split partials in scratch memory that the caller allocates.  Some
// callers cannot do that: a C program or another runtime's plugin that was handed a fixed slice
// of device memory at start-up and may not call cudaMalloc afterwards, or a latency-critical
// loop for which cudaMalloc's device-wide synchronisation is unacceptable.  For them the
// partials live in the array below, which is part of this library's image: every GPU that loads
// the library holds these 4 MiB until the process exits.
//
// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address;
// handing it to a kernel would fault or, where the GPU can reach host memory, quietly use the
// wrong bytes.  The device address is looked up once per device with cudaGetSymbolAddress while
// that device is current, and that pointer is what the kernel receives.
#include "attention_decode_noalloc.h"
#include <mutex>

static __device__ __align__(256) float g_noalloc_scratch[TB_ATTN_DECODE_NOALLOC_MAX_FLOATS];
// ticket counters of the split fold, one per (sequence, kv head); zero when the library is loaded and
// left at zero by every launch.  A call with more pairs than this folds with a second kernel instead.
#define NOALLOC_MAX_TICKETS 16384
static __device__ int g_noalloc_tickets[NOALLOC_MAX_TICKETS];

#define NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];          // device address of the array, per device
static int* g_noalloc_tickets_ptr[NOALLOC_MAX_DEVICES];
static std::mutex g_noalloc_mutex;

extern "C" int tb_attn_decode_noalloc(const DecodeArgs* args, int dtype, int batch, cudaStream_t stream) {
    if (batch <= 0) return 0;
    DecodeArgs a = *args;
    const long long need = a.n_splits > 1 ? (long long)batch * a.n_heads * a.n_splits * (a.hd + 2) : 0;
    if (need > (long long)TB_ATTN_DECODE_NOALLOC_MAX_FLOATS)
        return tb_refuse("attn_decode_noalloc: batch %d x %d heads x %d splits x (head_dim %d + 2) = %lld floats of "
                         "partials, the built-in scratch holds %lld; use fewer splits or tb_attn_decode with "
                         "scratch of your own", batch, a.n_heads, a.n_splits, a.hd, need,
                         (long long)TB_ATTN_DECODE_NOALLOC_MAX_FLOATS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return tb_refuse("attn_decode_noalloc: device index %d", dev);
    float* ptr;
    int* tickets;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_ptr[dev] == nullptr) {
            // set-up, once per device, with that device current
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess) return (int)e;
            void* t = nullptr;
            e = cudaGetSymbolAddress(&t, g_noalloc_tickets);
            if (e != cudaSuccess) return (int)e;
            g_noalloc_tickets_ptr[dev] = (int*)t;
            g_noalloc_ptr[dev] = (float*)p;
        }
        ptr = g_noalloc_ptr[dev];
        tickets = g_noalloc_tickets_ptr[dev];
    }
    a.partial = need ? ptr : nullptr;
    a.tickets = (need && (long long)batch * a.n_kv_heads <= NOALLOC_MAX_TICKETS) ? tickets : nullptr;
    return tb_attn_decode(&a, dtype, batch, stream);
}

// Reads and clears the error word (1: a bounded wait on a page copy ran out).  Synchronises.  A launch that
// gave up may have left its ticket counters half counted: the built-in counters of tb_attn_decode_noalloc are
// zeroed again here (the caller of tb_attn_decode zeroes its own).
extern "C" int tb_attn_decode_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) {
        cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
        void* t = nullptr;
        if (cudaGetSymbolAddress(&t, g_noalloc_tickets) == cudaSuccess && t != nullptr)
            cudaMemset(t, 0, sizeof(int) * NOALLOC_MAX_TICKETS);
    }
    return v;
}

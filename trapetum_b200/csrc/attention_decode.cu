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
// refused and the caller uses the generic kernel.  Two variants share the staging: the scalar
// one described above (tb_attn_decode_lanes) and the tensor-core one further down (tb_attn_decode,
// the product path).
#include "common.cuh"
#include "async.cuh"
#include <cuda.h>

TB_EXPORT_ERROR()

#define PAGE 64

__device__ int g_attn_error = 0;

struct DecodeArgs {
    const void* q; long long q_stride;
    const void* k_pool; const void* v_pool;
    const int* page_table; int pt_stride;
    const int* len_after;
    void* out;
    float* partial;
    int n_heads, n_kv_heads, hd, page_rows, ring_rows, window, n_splits;
    float scale, cap;
};

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
// Tensor-core variant: the group's query heads are the first rows of a 16-row MMA tile.
//
// Q.K^T and P.V run as mma.sync m16n8k16 (bfloat16 operands, 32-bit accumulators): per page of
// 64 keys a warp issues 64 MMAs instead of some 600 scalar instructions, so the kernel's time
// is the time of its page copies.  A page arrives as head_dim/64 tiled TMA copies of 64 keys x
// 64 dims with the 128-byte swizzle (8 KB each), the layout in which every ldmatrix is
// conflict-free; a dense copy would put all rows of a page on the same banks.  Each of the
// 4 warps owns 16 keys of a page for both products and keeps its own running softmax; the warps
// are folded at the end.  Rows of a page that are not keys of the sequence get their scores
// masked and their V rows zeroed in shared memory before use.
// ---------------------------------------------------------------------------
#define MW 4                                       // warps per CTA
template <int HD> struct MCfg {
    static constexpr int BOXES = HD / 64;                            // 64-dim column boxes per page
    static constexpr int BOX_BYTES = PAGE * 128;                     // 64 keys x 128 bytes, swizzled
    static constexpr int TILE_BYTES = BOXES * BOX_BYTES;             // one page of K (or V)
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int STAGES_RAW = (192 * 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment */ + 128;
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
// D += A B with rows 8..15 of A all zero (a1 = a3 = 0): only the group's heads occupy rows
__device__ __forceinline__ void mma_rows8(float* d, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t z = 0u;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}

template <int HD>
__global__ void __launch_bounds__(MW * 32, 1)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, DecodeArgs a) {
    pdl_launch_dependents();
    using C = MCfg<HD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
    __shared__ int s_abort;

    const int G = a.n_heads / a.n_kv_heads;                         // 1..8 query heads on rows 0..G-1
    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const int len = a.len_after[b];
    const int lo = (a.window > 0 && len > a.window) ? len - a.window : 0;
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

    // one thread issues the copies of a page: head_dim/64 boxes of K and as many of V
    auto issue = [&](int i) {
        const int s = i % C::STAGES;
        const int page = pt[pg_beg + i];
        const int row = (page * a.n_kv_heads + kvh) * PAGE;          // row of the pool seen as [rows, head_dim]
        uint8_t* dst = smem + s * C::STAGE_BYTES;
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
#pragma unroll
        for (int bx = 0; bx < C::BOXES; bx++) {
            tma_load_box(dst + bx * C::BOX_BYTES, &map_k, &full[s], bx * 64, row);
            tma_load_box(dst + C::TILE_BYTES + bx * C::BOX_BYTES, &map_v, &full[s], bx * 64, row);
        }
    };
    pdl_wait();                                     // the cache rows of this step and q come from earlier kernels
    if (threadIdx.x == 0)
        for (int i = 0; i < n && i < C::STAGES; i++) issue(i);

    // A fragments of Q: a0 = Q[g][16 ks + 2t, +1], a2 = Q[g][16 ks + 8 + 2t, +1]; rows >= G are zero
    uint32_t qa[HD / 16][2];
    {
        const bf16* qp = (const bf16*)a.q + (size_t)b * a.q_stride + (size_t)(kvh * G + g) * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            qa[ks][0] = (g < G) ? *(const uint32_t*)(qp + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = (g < G) ? *(const uint32_t*)(qp + ks * 16 + 8 + 2 * t) : 0u;
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run = -INFINITY, l_run = 0.f;                           // of row g (meaningful for g < G)

    // Which rows (in row space) are keys.  Without a ring, or before the ring has wrapped: lo <= R < len.
    // Once it has wrapped (len >= ring_rows) every row holds a token; too old are the ring_rows - window rows
    // that follow the newest one, a single circular run that starts at old_beg.
    const bool wrapped = a.ring_rows > 0 && len >= a.ring_rows;
    const int newest = wrapped ? (len - 1) % a.ring_rows : 0;
    const int n_old = wrapped ? a.ring_rows - a.window : 0;
    const int old_beg = wrapped ? (newest + 1 == a.ring_rows ? 0 : newest + 1) : 0;
    const bool no_invalid = wrapped && n_old == 0;                  // a full ring whose every row is in the window
    auto is_key = [&](int R) -> bool {
        if (wrapped) {
            int d = R - old_beg;                                    // distance past the start of the old run
            if (d < 0) d += a.ring_rows;
            return d >= n_old;
        }
        return R >= lo && R < len;
    };

    int consumed = 0;
    for (int i = 0; i < n; i++) {
        const int s = i % C::STAGES;
        const bool got = mbar_wait(&full[s], (i / C::STAGES) & 1);
        if (!__syncthreads_and(got)) { if (threadIdx.x == 0) s_abort = 1; break; }
        consumed = i + 1;
        uint8_t* k_s = smem + s * C::STAGE_BYTES;
        uint8_t* v_s = k_s + C::TILE_BYTES;
        const int key0 = warp * 16;                                  // this warp's keys within the page
        const int row0 = (pg_beg + i) * PAGE + key0;

        // ---- which of this warp's 16 rows are keys of the sequence
        bool all_ok;
        if (no_invalid) all_ok = true;
        else {
            all_ok = is_key(row0) && is_key(row0 + 15);
            // in a ring the rows that are too old form one circular run; it may lie inside these 16 rows
            if (wrapped && all_ok) all_ok = !(old_beg > row0 && old_beg <= row0 + 15);
        }
        if (!all_ok) {
            // zero the V rows that are not keys: p is 0 there, but 0 * NaN would still poison o
            for (int r = 0; r < 16; r++) {
                if (!is_key(row0 + r)) {
                    for (int c = lane; c < HD / 8; c += 32)
                        *(uint4*)(v_s + sw_off(key0 + r, c)) = make_uint4(0, 0, 0, 0);
                }
            }
            // these rows were written by ordinary stores; the stage is later refilled by bulk copies
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }

        // ---- S = Q K^T: 16 rows x 16 keys (two n-tiles)
        float sc[2][4], sc2[2][4];                                   // two chains per n-tile: even and odd k-steps
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) { sc[nt][e] = 0.f; sc2[nt][e] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(smem_u32(k_s + sw_off(key0 + (lane >> 4) * 8 + (lane & 7), ks * 2 + ((lane >> 3) & 1))), b0, b1, b2, b3);
            if (ks & 1) { mma_rows8(sc2[0], qa[ks][0], qa[ks][1], b0, b1); mma_rows8(sc2[1], qa[ks][0], qa[ks][1], b2, b3); }
            else { mma_rows8(sc[0], qa[ks][0], qa[ks][1], b0, b1); mma_rows8(sc[1], qa[ks][0], qa[ks][1], b2, b3); }
        }
#pragma unroll
        for (int nt = 0; nt < 2; nt++) { sc[nt][0] += sc2[nt][0]; sc[nt][1] += sc2[nt][1]; }
        // ---- scale, cap, mask; row g lives in sc[nt][0..1] of the quad's four lanes
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                float v = sc[nt][e] * a.scale;
                if (a.cap > 0.f) v = softcap_f(v, a.cap);
                const bool ok = all_ok || is_key(row0 + nt * 8 + 2 * t + e);
                v = ok ? v : -INFINITY;
                sc[nt][e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mn = fmaxf(m_run, mx);
        const float msafe = (mn == -INFINITY) ? 0.f : mn;
        const float corr = (m_run == -INFINITY) ? 0.f : __expf(m_run - msafe);
        m_run = mn;
        float p[2][2];
        float ps = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) { p[nt][e] = __expf(sc[nt][e] - msafe); ps += p[nt][e]; }
        l_run = l_run * corr + ps;
#pragma unroll
        for (int d = 0; d < HD / 8; d++) { o[d][0] *= corr; o[d][1] *= corr; }
        __nv_bfloat162 h0 = __floats2bfloat162_rn(p[0][0], p[0][1]), h1 = __floats2bfloat162_rn(p[1][0], p[1][1]);
        const uint32_t pa0 = (g < G) ? *(uint32_t*)&h0 : 0u, pa2 = (g < G) ? *(uint32_t*)&h1 : 0u;
        // ---- O += P V over this warp's 16 keys
#pragma unroll
        for (int d = 0; d < HD / 8; d += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(smem_u32(v_s + sw_off(key0 + ((lane >> 3) & 1) * 8 + (lane & 7), d + (lane >> 4))), b0, b1, b2, b3);
            mma_rows8(o[d], pa0, pa2, b0, b1);
            mma_rows8(o[d + 1], pa0, pa2, b2, b3);
        }
        __syncthreads();                                            // everyone is done with stage s
        if (threadIdx.x == 0 && i + C::STAGES < n) issue(i + C::STAGES);
    }

    if (s_abort) {
        if (threadIdx.x == 0) {
            atomicExch(&g_attn_error, 1);
            const int issued = min(n, consumed + C::STAGES);
            for (int i = consumed; i < issued; i++) mbar_wait(&full[i % C::STAGES], (i / C::STAGES) & 1);
        }
        __syncthreads();
        return;
    }

    // ---- fold the four warps: row sums over the quad first
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();
    float* red = (float*)smem;                                      // [MW][G][HD + 2]
    if (g < G) {
        float* r = red + ((size_t)warp * G + g) * (HD + 2);
#pragma unroll
        for (int d = 0; d < HD / 8; d++) { r[d * 8 + 2 * t] = o[d][0]; r[d * 8 + 2 * t + 1] = o[d][1]; }
        if (t == 0) { r[HD] = m_run; r[HD + 1] = l_run; }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < G * HD; x += blockDim.x) {
        const int gg = x / HD, d = x % HD;
        float M = -INFINITY;
        for (int w = 0; w < MW; w++) M = fmaxf(M, red[((size_t)w * G + gg) * (HD + 2) + HD]);
        float L = 0.f, acc = 0.f;
        for (int w = 0; w < MW; w++) {
            const float* r = red + ((size_t)w * G + gg) * (HD + 2);
            if (r[HD] != -INFINITY) { const float f = __expf(r[HD] - M); L += r[HD + 1] * f; acc += r[d] * f; }
        }
        const int h = kvh * G + gg;
        if (a.n_splits == 1) {
            ((bf16*)a.out)[((size_t)b * a.n_heads + h) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            float* pp = a.partial + (((size_t)b * a.n_heads + h) * a.n_splits + split) * (HD + 2);
            pp[d] = acc;
            if (d == 0) { pp[HD] = M; pp[HD + 1] = L; }
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

template <int HD>
static int launch_mma(const DecodeArgs& a, int batch, long long pool_rows, cudaStream_t stream) {
    using C = MCfg<HD>;
    static bool attr_set = false;
    auto kern = attn_decode_mma_kernel<HD>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    CUtensorMap mk, mv;
    if (pool_map(&mk, a.k_pool, pool_rows, HD) || pool_map(&mv, a.v_pool, pool_rows, HD)) return -1;
    dim3 grid(batch, a.n_kv_heads, a.n_splits);
    tb_launch(kern, dim3(grid), dim3(MW * 32), C::SMEM, stream, mk, mv, a);
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
    if (tensor_cores) {
        // the map's row count only bounds the copy engine's address check; pages come from the table
        const long long rows = 0x7fffff00LL;
        switch (a.hd) {
        case 64: st = launch_mma<64>(a, batch, rows, stream); break;
        case 128: st = launch_mma<128>(a, batch, rows, stream); break;
        default: st = launch_mma<256>(a, batch, rows, stream); break;
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
    if (a.n_splits > 1) {
        tb_launch(attn_combine_kernel, dim3((unsigned)batch * a.n_heads), dim3(128), 0, stream, a.partial, (bf16*)a.out, a.n_splits, a.hd);
        st = tb_launch_status();
    }
    return st;
}

// Reads and clears the error word (1: a bounded wait on a page copy ran out).  Synchronises.
extern "C" int tb_attn_decode_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
    return v;
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

#define NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];          // device address of the array, per device
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
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_ptr[dev] == nullptr) {
            // set-up, once per device, with that device current
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess) return (int)e;
            g_noalloc_ptr[dev] = (float*)p;
        }
        ptr = g_noalloc_ptr[dev];
    }
    a.partial = need ? ptr : nullptr;
    return tb_attn_decode(&a, dtype, batch, stream);
}

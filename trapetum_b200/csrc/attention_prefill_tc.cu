// Prefill attention on the 5th-generation tensor cores (tcgen05, bfloat16): causal, packed sequences
// of unequal length, optional sliding window and tanh soft cap, grouped-query heads.
//
// Same formula as attention_prefill.cu (and as the reference's one-query attn_k,
// runtime/cuda/codebook_gemv.cu:240-270); what differs is where the work runs:
//   * one CTA = 128 queries of one head of one sequence; S = Q K^T and O += P V are tcgen05.mma
//     (128 x 64 x 16 and 128 x head_dim x 16) issued by one thread, with S and O in tensor memory;
//   * tensor memory's lanes are the query rows, so a row's running maximum, exponentials and row sum
//     stay with the row's threads: no shuffles across a warp;
//   * K and V tiles arrive by tiled TMA (128-byte swizzle); P is written to shared
//     memory in the same swizzled K-major layout and is the A operand of the second product;
//   * Q lies in tensor memory (each softmax thread loads its row once) and is the first product's A operand
//     from there: the tensor core would otherwise read the whole Q tile from shared memory again for every
//     key block, and shared-memory bandwidth (operand reads, TMA writes, P) is what bounds a block's time;
//   * the exponent's reference maximum is only raised when a block's maximum exceeds it by 2^8
//     ("lazy rescaling"): then the thread scales its O row in tensor memory; otherwise O is left
//     alone and p may reach 256, which bfloat16 and the 32-bit accumulators hold without loss;
//   * warp 0 loads, warp 1 issues MMAs, warps 2..9 are the softmax: two groups of four warps, one thread per
//     row each; the first group takes the even key blocks, the second the odd ones, so two blocks' softmax run
//     at a time (S and P are double-buffered) and one group's waits (for S, for tensor memory, for the P buffer)
//     are covered by the other's exponentials.  A row's two threads hand its reference maximum back and forth
//     through shared memory: the only thing block j+1 needs from block j.
// V is the second product's B operand as it lies in memory, [key][dim] with the dims contiguous ("MN-major": the
// descriptor's leading-dimension offset is the distance between panels of 64 dims, its stride offset the distance
// between groups of 8 keys), so no transposed copy of V is made.  Keys past a sequence's end are the next
// sequence's rows or, past the last token, the zeros that TMA fills in; their P is zero.
//
// All waits are bounded (async.cuh); a wait that runs out records an error word.
// Compiled once per head size (-DTB_HD = 64, 128 or 256).
#include "common.cuh"
#include "tcgen05.cuh"

TB_EXPORT_ERROR()

#ifndef TB_HD
#define TB_HD 256
#endif
constexpr int HD = TB_HD;
static_assert(HD == 64 || HD == 128 || HD == 256, "head_dim 64, 128 or 256");
#define BM 128
#define BN 64
constexpr int QBOXES = HD / 64;                       // 64-dim boxes along the head dim
constexpr int K_BYTES = QBOXES * BN * 128;            // 64 keys x head_dim
constexpr int V_BYTES = K_BYTES;                      // 64 keys x head_dim, as K
constexpr int P_BYTES = BM * 128;                     // 128 rows x 64 keys
constexpr int TILE_BYTES = 2 * K_BYTES + 2 * V_BYTES + 2 * P_BYTES;
constexpr int ROWX_BYTES = 2 * 2 * BM * 4;         // the softmax threads' exchange: references [2][BM], row sums [2][BM]
constexpr int USED_BYTES = TILE_BYTES + ROWX_BYTES + 256;
constexpr int SMEM_BYTES = USED_BYTES + 512;       // head_dim 256 uses all but 256 bytes of an SM's shared memory
static_assert(SMEM_BYTES <= 232448, "does not fit an SM's shared memory");
constexpr int Q_COLS = HD / 2;                        // Q in tensor memory: two bf16 per column
constexpr int TMEM_COLS = (2 * BN + HD + Q_COLS) <= 256 ? 256 : 512;
static_assert(2 * BN + HD + Q_COLS <= 512, "tensor memory holds S twice, O and Q");
constexpr float RESCALE_AT = 8.f;                     // in log2 units

__device__ int g_attn_tc_error = 0;

struct PrefillTcArgs {
    const bf16* q;                 // [T, q_stride]: head h of token t at q + t * q_stride + h * HD
    long long q_stride;
    int n_tokens;
    const int* seq_start;          // [B + 1] rows of the packed q/k matrices
    bf16* out;                     // [T, n_heads * HD]
    int n_heads, n_kv_heads, window;
    float scale, cap;
};

__device__ __forceinline__ float ex2f(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcpf(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__global__ void __launch_bounds__(320, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, PrefillTcArgs a) {
    pdl_launch_dependents();
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    if (smem + USED_BYTES > smem_raw + SMEM_BYTES) {                 // the base was less aligned than assumed
        if (threadIdx.x == 0) atomicExch(&g_attn_tc_error, 4);
        return;
    }
    uint8_t* sK = smem;                               // [2][K_BYTES]
    uint8_t* sV = sK + 2 * K_BYTES;                   // [2][V_BYTES]
    uint8_t* sP = sV + 2 * V_BYTES;                   // [2][P_BYTES]
    float (*row_ref)[BM] = (float (*)[BM])(sP + 2 * P_BYTES);        // [block parity][row]: the reference after that block
    float (*row_l)[BM] = row_ref + 2;                                // [group][row]: the groups' row sums at the end
    uint64_t* bars = (uint64_t*)(sP + 2 * P_BYTES + ROWX_BYTES);
    uint64_t* q_full = bars;                          // 1
    uint64_t* k_full = bars + 1;                      // [2]
    uint64_t* k_empty = bars + 3;                     // [2]
    uint64_t* v_full = bars + 5;                      // [2]
    uint64_t* v_empty = bars + 7;                     // [2]  (also: P buffer free)
    uint64_t* s_full = bars + 9;                      // [2]
    uint64_t* s_empty = bars + 11;                    // [2]
    uint64_t* p_full = bars + 13;                     // [2]
    uint64_t* x_bar = bars + 15;                      // 1: the softmax groups meet at the end
    uint64_t* ref_full = bars + 16;                   // [2]: block j's reference is in row_ref[j & 1]
    uint32_t* tmem_slot = (uint32_t*)(bars + 18);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y, h = blockIdx.x;
    const int s0 = a.seq_start[b], len = a.seq_start[b + 1] - s0;
    // Blocks are placed in the order of their index, x fastest: the heads of one query block side by side (those of a
    // kv head read the same keys), then the sequences; the longest query blocks of every head and sequence first.
    const int qb = (int)gridDim.z - 1 - (int)blockIdx.z;
    const int m0 = qb * BM;
    if (m0 >= len) return;                                           // uniform for the CTA
    const int kvh = h / (a.n_heads / a.n_kv_heads);

    // key blocks this query block can see
    const int i_last = min(len, m0 + BM) - 1;
    const int j_lo = (a.window > 0) ? max(0, m0 - a.window + 1) : 0;
    const int nb_lo = j_lo / BN, nb_hi = i_last / BN + 1;
    const int nblocks = nb_hi - nb_lo;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 8);
        for (int s = 0; s < 2; s++) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 4); mbar_init(&p_full[s], 4); mbar_init(&ref_full[s], 4);
        }
        mbar_init(x_bar, 8);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    if (threadIdx.x == 64) { tma_prefetch_map(&map_k); tma_prefetch_map(&map_v); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base;                               // [2][BN] columns
    const uint32_t tmem_o = tmem_base + 2 * BN;                      // HD columns
    const uint32_t tmem_q = tmem_o + HD;                             // Q_COLS columns

    if (warp == 0) {
        // ---------------- loads, and the second product's MMAs ----------------
        // (One thread can issue an MMA every fifty cycles or so; the first product's MMAs run no longer than that.
        //  So the two products have an issuing thread each, and neither waits behind the other's operands.)
        if (lane == 0) {
            pdl_wait();
            constexpr uint32_t idesc_o = instr_desc(HD) | (1u << 16);           // B (= V) is MN-major
            const uint32_t hi = desc_hi(smem_desc(0));
            const uint32_t p_lo0 = desc_lo(smem_desc(smem_u32(sP)));
            // V: panels of 64 dims lie BN * 128 bytes apart (leading-dimension offset, bits 16..29 of the low half);
            // groups of 8 keys 1024 bytes apart, which is the stride offset that the K-major operands have too
            const uint32_t v_lo0 = ((smem_u32(sV) & 0x3ffff) >> 4) | ((uint32_t)((BN * 128) >> 4) << 16);
            bool ok = true;
            // K tiles, V^T tiles and the second products are started independently, each as soon as it has what it
            // needs: the scores run up to two blocks ahead of the second product, and so must the K tiles
            int jk = 0, jv = 0, jp = 0;
            long long idle_since = clock64();
            while (ok && jp < nblocks) {
                bool moved = false;
                if (jk < nblocks && mbar_test(&k_empty[jk & 1], ((jk >> 1) & 1) ^ 1)) {
                    const int s = jk & 1, key0 = (nb_lo + jk) * BN;
                    mbar_expect_tx(&k_full[s], K_BYTES);
                    for (int c = 0; c < QBOXES; c++)
                        tma_load_2d(sK + s * K_BYTES + c * BN * 128, &map_k, &k_full[s], kvh * HD + c * 64, s0 + key0);
                    jk++; moved = true;
                }
                if (jv < nblocks && mbar_test(&v_empty[jv & 1], ((jv >> 1) & 1) ^ 1)) {
                    const int s = jv & 1, key0 = (nb_lo + jv) * BN;
                    mbar_expect_tx(&v_full[s], V_BYTES);
                    for (int c = 0; c < QBOXES; c++)
                        tma_load_2d(sV + s * V_BYTES + c * BN * 128, &map_v, &v_full[s], kvh * HD + c * 64, s0 + key0);
                    jv++; moved = true;
                }
                if (mbar_test(&v_full[jp & 1], (jp >> 1) & 1) && mbar_test(&p_full[jp & 1], (jp >> 1) & 1)) {
                    const int s = jp & 1;
                    tc_fence_after();
                    const uint32_t p_lo = p_lo0 + s * (P_BYTES >> 4), v_lo = v_lo0 + s * (V_BYTES >> 4);
#pragma unroll
                    for (int ks = 0; ks < BN / UMMA_K; ks++)          // 16 keys on: 32 bytes in a row of P, 16 rows of V
                        umma_bf16_lh(tmem_o, p_lo + ks * 2, v_lo + ks * ((UMMA_K * 128) >> 4), hi, idesc_o,
                                     (jp > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(&v_empty[s]);         // V tile and P buffer are free again; O holds blocks 0..jp
                    jp++; moved = true;
                }
                if (moved) idle_since = clock64();
                else if (*abort_flag || clock64() - idle_since > WAIT_CYCLES) ok = false;
            }
            if (!ok && !*abort_flag) { atomicExch(&g_attn_tc_error, 1); *abort_flag = 1; }
        }
    } else if (warp == 1) {
        // ---------------- the first product's MMAs ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(BN);
            const uint32_t hi = desc_hi(smem_desc(0));
            const uint32_t k_lo0 = desc_lo(smem_desc(smem_u32(sK)));
            bool ok = mbar_wait(q_full, 0);
            // the scores of block j + 2 are issued when S of block j has been read, long before P of block j exists:
            // the softmax does not wait for them
            for (int j = 0; j < nblocks && ok; j++) {
                const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
                if (*abort_flag || !mbar_wait(&k_full[s], ph) || !mbar_wait(&s_empty[s], ph ^ 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t k_lo = k_lo0 + s * (K_BYTES >> 4), d = tmem_s + s * BN;
#pragma unroll
                for (int ks = 0; ks < HD / UMMA_K; ks++)
                    umma_bf16_ta_lh(d, tmem_q + ks * (UMMA_K / 2), k_lo + (((ks >> 2) * (BN * 128) + (ks & 3) * 32) >> 4), hi,
                                    idesc_s, ks > 0 ? 1u : 0u);
                umma_commit(&k_empty[s]);             // K tile may be overwritten once these have run
                umma_commit(&s_full[s]);              // and S is ready for the softmax
            }
            if (!ok && !*abort_flag) { atomicExch(&g_attn_tc_error, 2); *abort_flag = 1; }
        }
    } else {
        // ---------------- softmax: one thread per query row and group; group g takes the blocks j = g, g + 2, .. ----------------
        const int sw = warp - 2;                                     // 0..7
        const int quarter = warp & 3;                                // the TMEM lanes this warp may touch
        const int group = sw >> 2;
        const int r = quarter * 32 + lane;                           // row of the tile = TMEM lane
        const int i = m0 + r;                                        // position of the query in its sequence
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float LOG2E = 1.4426950408889634f;
        const float sc2 = a.scale * LOG2E;                           // scores in log2 units
        const float cap2 = a.cap * LOG2E;
        const float cap_k = a.cap > 0.f ? 2.f * a.scale / a.cap * LOG2E : 0.f;
        float m_ref = -INFINITY, l_sum = 0.f;                        // this thread's reference and its share of the row sum
        bool ok = true;
        pdl_wait();
        {
            // this thread's query row into tensor memory (rows past the last token: zeros); with head sizes from 128
            // the two threads of a row take half of it each
            constexpr int PER = (Q_COLS >= 64) ? Q_COLS / 2 : Q_COLS;            // columns per thread that loads
            const long long row = (long long)s0 + i;
            const bool inside = row < a.n_tokens;
            if (Q_COLS >= 64 || group == 0) {
                const int col0 = (Q_COLS >= 64) ? group * PER : 0;
                const uint4* src = (const uint4*)(a.q + row * a.q_stride + (size_t)h * HD + col0 * 2);
#pragma unroll 1
                for (int c0 = 0; c0 < PER; c0 += 32) {
                    uint32_t w[32];
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const uint4 x = inside ? __ldg(src + c0 / 4 + k) : make_uint4(0u, 0u, 0u, 0u);
                        w[4 * k] = x.x; w[4 * k + 1] = x.y; w[4 * k + 2] = x.z; w[4 * k + 3] = x.w;
                    }
                    tmem_st32(tmem_q + lane_addr + col0 + c0, w);
                }
                tmem_st_wait();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        for (int j = group; j < nblocks; j += 2) {
            const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
            const bool got = !*abort_flag && mbar_wait(&s_full[s], ph);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
            tc_fence_after();
            float v[BN];
            tmem_ld32(tmem_s + s * BN + lane_addr, (uint32_t*)v);
            tmem_ld32(tmem_s + s * BN + lane_addr + 32, (uint32_t*)v + 32);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[s]);                 // this warp has read its part of S
            // scale, cap, mask; values in log2 units
            const int key0 = (nb_lo + j) * BN;
            const bool edge = (key0 + BN - 1 > m0) || (key0 + BN > len) || (a.window > 0 && (m0 + BM - 1) - key0 >= a.window);
            if (a.cap > 0.f) {
                // cap * tanh(x * scale / cap) = cap - 2 cap / (e^(2 x scale / cap) + 1), in log2 units; 2^(+big) is
                // inf and its reciprocal 0, 2^(-big) is 0: both ends come out right without a clamp
#pragma unroll
                for (int c = 0; c < BN; c++) v[c] = fmaf(-2.f * cap2, rcpf(ex2f(v[c] * cap_k) + 1.f), cap2);
            } else {
#pragma unroll
                for (int c = 0; c < BN; c++) v[c] *= sc2;
            }
            if (edge) {
#pragma unroll
                for (int c = 0; c < BN; c++) {
                    const int jj = key0 + c;
                    if (!(jj <= i && jj < len && (a.window <= 0 || i - jj < a.window))) v[c] = -INFINITY;
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < BN; c += 4)
                mx = fmaxf(mx, fmaxf(fmaxf(v[c], v[c + 1]), fmaxf(v[c + 2], v[c + 3])));
            // the row's reference after block j-1, from the other group (a bounded mbarrier wait: no wait here may hang)
            float before = -INFINITY;
            if (j > 0) {
                const bool met = mbar_wait(&ref_full[(j - 1) & 1], ((j - 1) >> 1) & 1);
                if (!__all_sync(0xffffffffu, met)) { ok = false; break; }
                before = row_ref[(j - 1) & 1][r];
            }
            if (before != m_ref) {                                   // the other group raised it: this share follows
                l_sum *= (m_ref == -INFINITY) ? 0.f : ex2f(m_ref - before);
                m_ref = before;
            }
            // lazy rescaling: raise the reference only when the block's maximum is far above it
            float factor = 1.f;
            bool raise = mx > m_ref + RESCALE_AT;
            if (m_ref == -INFINITY) raise = mx != -INFINITY;         // first block with a visible key
            if (raise) {
                factor = (m_ref == -INFINITY) ? 0.f : ex2f(m_ref - mx);
                m_ref = mx;
            }
            row_ref[j & 1][r] = m_ref;
            __syncwarp();
            if (lane == 0) mbar_arrive(&ref_full[j & 1]);
            const float mr = (m_ref == -INFINITY) ? 0.f : m_ref;
            uint32_t pk[BN / 2];
            float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                const float p0 = ex2f(v[c] - mr), p1 = ex2f(v[c + 1] - mr);
                ls0 += p0; ls1 += p1;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                pk[c >> 1] = *(uint32_t*)&h2;
            }
            l_sum = l_sum * factor + (ls0 + ls1);
            // O holds the blocks before j: scale this row if its reference moved (not for the first block: the
            // second product starts O from zero).
            const bool need = raise && j > 0;
            if (__any_sync(0xffffffffu, need)) {
                // every MMA into O must have completed: block j-1's second product signals v_empty of its slot
                // (block j-3's has for certain, since S of block j is there, so the parity is unambiguous)
                const bool done = mbar_wait(&v_empty[(j - 1) & 1], ((j - 1) >> 1) & 1);
                if (!__all_sync(0xffffffffu, done)) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem_o + lane_addr + c0, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; e++) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * factor);
                    tmem_st32(tmem_o + lane_addr + c0, ov);
                }
                tmem_st_wait();
            }
            // P into shared memory (free once the second product of block j-2 has run)
            const bool freep = mbar_wait(&v_empty[s], ph ^ 1);
            if (!__all_sync(0xffffffffu, freep)) { ok = false; break; }
            uint8_t* prow = sP + s * P_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < 8; c++)
                *(uint4*)(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // visible to the tensor core's reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[s]);
        }
        if (ok) {
            // ---- the last product has to land, then O / l goes out
            const bool done = mbar_wait(&v_empty[(nblocks - 1) & 1], ((nblocks - 1) >> 1) & 1);
            ok = __all_sync(0xffffffffu, done);
        }
        if (ok) {
            // both shares of the row sum at the row's last reference
            const int last = nblocks - 1;
            if ((last & 1) != group) {
                const bool met = mbar_wait(&ref_full[last & 1], (last >> 1) & 1);
                ok = __all_sync(0xffffffffu, met);
                if (ok) {
                    const float fin = row_ref[last & 1][r];
                    if (fin != m_ref) l_sum *= (m_ref == -INFINITY) ? 0.f : ex2f(m_ref - fin);
                }
            }
        }
        if (ok) {
            row_l[group][r] = l_sum;
            __syncwarp();
            if (lane == 0) mbar_arrive(x_bar);
            const bool met = mbar_wait(x_bar, 0);
            ok = __all_sync(0xffffffffu, met);
        }
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / (row_l[0][r] + row_l[1][r]);
            bf16* orow = a.out + ((size_t)(s0 + i) * a.n_heads + h) * HD;
#pragma unroll 1
            for (int c0 = group * (HD / 2); c0 < (group + 1) * (HD / 2); c0 += 32) {   // each group writes half of the columns
                uint32_t ov[32];
                tmem_ld32(tmem_o + lane_addr + c0, ov);
                tmem_ld_wait();
                if (i < len) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(ov[e + 2 * k]) * inv,
                                                                      __uint_as_float(ov[e + 2 * k + 1]) * inv);
                            w[k] = *(uint32_t*)&h2;
                        }
                        *(uint4*)(orow + c0 + e) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
        if (!ok && !*abort_flag && lane == 0) { atomicExch(&g_attn_tc_error, 3); *abort_flag = 1; }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
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
static int make_map(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return tb_refuse("attn_prefill_tc: the driver does not provide cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return tb_refuse("attn_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

extern "C" int tb_attn_prefill_tc_head_dim() { return HD; }

extern "C" int tb_attn_prefill_tc(const void* q, const void* k, const void* v, long long q_stride, long long kv_stride,
                                  const int* seq_start, void* out, int n_tokens, int batch, int max_seq_len, int n_heads,
                                  int n_kv_heads, int hd, float scale, float cap, int window, cudaStream_t stream) {
    if (batch <= 0 || max_seq_len <= 0) return 0;
    if (hd != HD) return tb_refuse("attn_prefill_tc: this library is built for head_dim %d, got %d", HD, hd);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads)
        return tb_refuse("attn_prefill_tc: %d heads cannot share %d kv heads", n_heads, n_kv_heads);
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || (q_stride % 8) || (kv_stride % 8))
        return tb_refuse("attn_prefill_tc: q, k, v rows must be 16-byte aligned");
    if ((max_seq_len + BM - 1) / BM > 65535 || batch > 65535)
        return tb_refuse("attn_prefill_tc: %d query blocks x %d sequences exceed one launch", (max_seq_len + BM - 1) / BM, batch);
    const int kvw = n_kv_heads * HD;
    CUtensorMap mk, mv;
    if (make_map(&mk, k, n_tokens, kvw, kv_stride, BN) || make_map(&mv, v, n_tokens, kvw, kv_stride, BN)) return -1;
    PrefillTcArgs a;
    a.q = (const bf16*)q; a.q_stride = q_stride; a.n_tokens = n_tokens;
    a.seq_start = seq_start; a.out = (bf16*)out;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.window = window; a.scale = scale; a.cap = cap;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    dim3 grid(n_heads, batch, (max_seq_len + BM - 1) / BM);
    tb_launch(attn_prefill_tc_kernel, grid, dim3(320), SMEM_BYTES, stream, mk, mv, a);
    return tb_launch_status();
}

extern "C" int tb_attn_prefill_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    return v;
}

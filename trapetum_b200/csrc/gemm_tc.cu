// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores.
//
// tcgen05.mma (kind::f16; cta_group::1 with 128 x BN x 16 per instruction, and for long
// products of many tokens cta_group::2 with 256 x 256 x 16 over a pair of SMs, see
// gemm_tc_pair_kernel) issued by one thread, operands staged in shared memory by TMA
// (128-byte swizzle, K-major), accumulators in tensor memory, read back with tcgen05.ld
// for the epilogue.
// The reference has no dense tensor-core product: its linears are 4-bit codebook
// GEMVs (runtime/cuda/codebook_gemv.cu:86-114) with a fixed-order second stage
// for determinism (:178-184); the same rule holds here (no atomics anywhere).
//
// One kernel, two orientations, chosen by the host:
//   tokens >  128: the 128 lanes of a tile are tokens, its BN columns weight rows
//   tokens <= 128: swapped, the 128 lanes are weight rows and the BN columns are the
//                  tokens (BN = 16..128), so a decode step streams every weight
//                  once through full-height MMA tiles whatever the batch size
// and optional split-K (small N, large K): each split writes 32-bit partials to
// scratch and tb_splitk_reduce adds them in split order.
//
// Roles per CTA (320 threads): warp 0 issues TMA loads, warp 1 owns tensor memory
// and issues the MMAs, warps 2..9 are the epilogue (a warp reads the 32 lanes of
// tensor memory that its index modulo 4 selects; the two warps of a quarter take
// the chunks of columns in turn).  The kernel is persistent: a
// CTA walks its share of the work items; two accumulator stages let the epilogue
// of one item overlap the MMAs of the next.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records a code in
// the error word, and all roles leave their loops, wait (bounded) for TMA loads
// still in flight, free the tensor memory and return.  tb_gemm_tc_error() reads
// and clears the word.
//
// Sizes: K must be a multiple of 8 elements and A, W 16-byte aligned (TMA strides);
// anything else is refused and the caller falls back to the FMA kernel.
#include "common.cuh"
#include "tcgen05.cuh"
#include <stdlib.h>

TB_EXPORT_ERROR()

#define BM 128
#define BK 64
#define EPI_WARPS 8                      // two warps for each quarter of the tensor memory's lanes
#define GEMM_THREADS (64 + 32 * EPI_WARPS)

__device__ int g_gemm_error = 0;

// ---------------------------------------------------------------------------
struct GemmParams {
    int rows_p, rows_q, K;           // P: the 128-lane operand, Q: the BN-column operand
    int tiles_p, tiles_q, splits, kb_per_split, kblocks;
    void* out; long long ld_out;     // C as [tokens, weight rows], row stride ld_out
    float* partial;                  // [splits][tokens][weight rows] when splits > 1
    float cap;
    int act;                         // gated epilogue: 0 gelu_tanh, 1 silu (only with GATED kernels)
};

// Gated epilogue.  The weight rows are interleaved in blocks of 16: [gate 0..15 | up 0..15 | gate 16..31 | ...],
// so that a gate and its up value always meet in one epilogue thread (token-major tiles: columns j and j + 16
// of a 32-column chunk) or in one warp (swapped tiles: lanes l and l + 16).  The output has half the width:
// out[token][16 b + j] = act(gate) * up, computed on the 32-bit accumulators
// (the reference's gelu_mul_k does this as a kernel of its own, runtime/cuda/codebook_gemv.cu:531-537).
// The result is rounded to bfloat16, so tanh and the logistic function are taken through the fast exponential
// and division (relative error near 2^-21): 0.5 (1 + tanh(y)) = 1 / (1 + e^(-2y)).
__device__ __forceinline__ float gated(float g, float u, int act) {
    const float y = act == 0 ? 1.5957691216f * (g + 0.044715f * g * g * g) : g;     // 2 sqrt(2/pi) (g + 0.044715 g^3)
    return __fdividef(g, 1.0f + __expf(-y)) * u;
}

// Shared-memory budget.  Many tokens (tiles are reused, the tensor cores are the limit): as many stages as an SM
// holds.  Few tokens (swapped tiles, a stream of weights) and a short stream: half of an SM, so that the next
// product's CTAs already sit beside this one's, fetch their tensor maps and fill their stages with weights while this
// one drains; the two kernels together keep as many bytes in flight as one with the whole SM.  A long stream (WIDE:
// the host asks for it from TB_WIDE_FROM_BYTES of weights on) takes the whole SM: its own bytes in flight count for
// more than the overlap with its neighbours.  Measured, decode steps at context 2,048 with every small product on
// the whole SM against half: 2B shape 2.5 % slower at batch 8, 9B shape 2 % faster, 27B shape 5 % faster; with 32 to
// 128 tokens the whole SM is never slower (9B shape at batch 64: 4 % faster).
#ifndef TB_SWAP_KB
#define TB_SWAP_KB 108
#endif
#ifndef TB_WIDE_FROM_BYTES
#define TB_WIDE_FROM_BYTES (128 << 20)
#endif
#ifndef TB_SWAP_HALF_UPTO
#define TB_SWAP_HALF_UPTO 16
#endif
template <int BN, bool SWAP, bool WIDE = false> struct Cfg {
    static constexpr int STAGE_BYTES = BM * BK * 2 + BN * BK * 2;
    static constexpr int BUDGET = ((SWAP && !WIDE && BN <= TB_SWAP_HALF_UPTO) ? TB_SWAP_KB : 200) * 1024;
    static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;               // columns of one accumulator stage
    static constexpr int TMEM_COLS = 2 * ACC_COLS;                   // a power of two >= 32
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
};

// Epilogue of token-major tiles: the thread holds CH consecutive columns (weight rows q0 .. q0 + CH - 1) of token prow.
template <typename TOut, bool GATED, int CH>
__device__ __forceinline__ void store_token_major(const uint32_t* r, int prow, int q0, int sp, const GemmParams& p) {
    static_assert(!GATED || CH == 32, "a gate and its up value lie 16 columns apart");
    if (GATED) {
        // 32 columns = 16 gates then their 16 ups: 16 outputs at column q0 / 2
        if (prow < p.rows_p && q0 < p.rows_q) {
            bf16* dst = (bf16*)p.out + (size_t)prow * p.ld_out + (q0 >> 1);
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const float v0 = gated(__uint_as_float(r[j]), __uint_as_float(r[j + 16]), p.act);
                const float v1 = gated(__uint_as_float(r[j + 1]), __uint_as_float(r[j + 17]), p.act);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
                w[j >> 1] = *(uint32_t*)&h2;
            }
            if ((((uintptr_t)dst) & 15) == 0) {
                *(uint4*)dst = make_uint4(w[0], w[1], w[2], w[3]);
                *(uint4*)(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) *(uint32_t*)(dst + 2 * j) = w[j];
            }
        }
    } else {
        // tokens on lanes (prow), weight rows on columns (q0 + j): a thread writes a row segment
        if (prow < p.rows_p) {
            if (p.splits > 1) {
                float* dst = p.partial + ((size_t)sp * p.rows_p + prow) * p.rows_q + q0;
#pragma unroll
                for (int j = 0; j < CH; j++) if (q0 + j < p.rows_q) dst[j] = __uint_as_float(r[j]);
            } else {
                TOut* dst = (TOut*)p.out + (size_t)prow * p.ld_out + q0;
                const bool vec = (q0 + CH <= p.rows_q) && ((((uintptr_t)dst) & 15) == 0);
                if (vec && sizeof(TOut) == 2) {
#pragma unroll
                    for (int j = 0; j < CH; j += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float v0 = __uint_as_float(r[j + 2 * e]), v1 = __uint_as_float(r[j + 2 * e + 1]);
                            if (p.cap > 0.f) { v0 = softcap_f(v0, p.cap); v1 = softcap_f(v1, p.cap); }
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
                            w[e] = *(uint32_t*)&h2;
                        }
                        *(uint4*)((bf16*)dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else if (vec) {
#pragma unroll
                    for (int j = 0; j < CH; j += 4) {
                        float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                               __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        if (p.cap > 0.f) { v.x = softcap_f(v.x, p.cap); v.y = softcap_f(v.y, p.cap);
                                           v.z = softcap_f(v.z, p.cap); v.w = softcap_f(v.w, p.cap); }
                        *(float4*)((float*)dst + j) = v;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < CH; j++) if (q0 + j < p.rows_q) {
                        float v = __uint_as_float(r[j]);
                        if (p.cap > 0.f) v = softcap_f(v, p.cap);
                        dst[j] = from_f<TOut>(v);
                    }
                }
            }
        }
    }
}

template <int BN, bool SWAP, typename TOut, bool GATED, bool WIDE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, GemmParams p) {
    pdl_launch_dependents();
    using C = Cfg<BN, SWAP, WIDE>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* full = bars;                       // [STAGES]
    uint64_t* empty = bars + C::STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * C::STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;          // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 32) { tma_prefetch_map(&map_p); tma_prefetch_map(&map_q); }
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; a++) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], EPI_WARPS); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_items = p.tiles_p * p.tiles_q * p.splits;
    // item -> (tile_q, tile_p, split): the tiles that share a Q tile (prefill: a weight
    // tile; swapped: the tokens) run side by side
    auto decode = [&](int item, int& tp, int& tq, int& sp) {
        sp = item % p.splits; item /= p.splits;
        tp = item % p.tiles_p; tq = item / p.tiles_p;
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true, waited = false;
            // the tile that holds weights: the 128-lane operand when swapped, else the BN-column one
            const CUtensorMap* wmap = SWAP ? &map_p : &map_q;
            const CUtensorMap* amap = SWAP ? &map_q : &map_p;
            constexpr int W_OFF = SWAP ? 0 : BM * BK * 2, A_OFF = SWAP ? BM * BK * 2 : 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int tp, tq, sp; decode(item, tp, tq, sp);
                const int kb0 = sp * p.kb_per_split, kb1 = min(p.kblocks, kb0 + p.kb_per_split);
                const int w_row = SWAP ? tp * BM : tq * BN, a_row = SWAP ? tq * BN : tp * BM;
                int kb = kb0;
                if (!waited) {
                    // Weights do not depend on the kernel before this one: start streaming them into the
                    // (still empty) stages at once, and only then wait for that kernel, whose output is
                    // the activation operand.
                    const int pre = min(kb1 - kb0, C::STAGES);
                    for (int j = 0; j < pre; j++) {
                        mbar_expect_tx(&full[j], C::STAGE_BYTES);
                        tma_load_2d(smem + j * C::STAGE_BYTES + W_OFF, wmap, &full[j], (kb0 + j) * BK, w_row);
                    }
                    pdl_wait();
                    waited = true;
                    for (int j = 0; j < pre; j++)
                        tma_load_2d(smem + j * C::STAGE_BYTES + A_OFF, amap, &full[j], (kb0 + j) * BK, a_row);
                    it = pre; kb = kb0 + pre;
                }
                for (; kb < kb1; kb++, it++) {
                    const int s = it % C::STAGES; const uint32_t ph = (it / C::STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) { ok = false; break; }
                    uint8_t* st = smem + s * C::STAGE_BYTES;
                    mbar_expect_tx(&full[s], C::STAGE_BYTES);
                    tma_load_2d(st + W_OFF, wmap, &full[s], kb * BK, w_row);
                    tma_load_2d(st + A_OFF, amap, &full[s], kb * BK, a_row);
                }
            }
            if (!ok) {
                if (!*abort_flag) { atomicExch(&g_gemm_error, 1); *abort_flag = 1; }
                // loads already issued still land in this CTA's shared memory: wait for them
                for (uint32_t back = 1; back <= (uint32_t)C::STAGES && back <= it; back++) {
                    const uint32_t j = it - back;
                    mbar_wait(&full[j % C::STAGES], (j / C::STAGES) & 1);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, tile_it++) {
                int tp, tq, sp; decode(item, tp, tq, sp);
                const int kb0 = sp * p.kb_per_split, kb1 = min(p.kblocks, kb0 + p.kb_per_split);
                const int a = tile_it & 1; const uint32_t aph = (tile_it >> 1) & 1;
                if (*abort_flag || !mbar_wait(&acc_empty[a], aph ^ 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_addr = tmem_base + a * C::ACC_COLS;
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % C::STAGES; const uint32_t ph = (it / C::STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&full[s], ph)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
                    const uint32_t sb = sa + BM * BK * 2;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        umma_bf16(d_addr, smem_desc(sa + k * UMMA_K * 2), smem_desc(sb + k * UMMA_K * 2), idesc,
                                  (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);            // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[a]);     // the accumulator is complete
            }
            if (!ok && !*abort_flag) { atomicExch(&g_gemm_error, 2); *abort_flag = 1; }
        }
    } else {
        // ---------------- epilogue: warps 2..9 ----------------
        const int quarter = warp & 3;                  // the TMEM lanes this warp may read
        const int turn = (warp - 2) >> 2;              // the two warps of a quarter take the chunks of columns in turn
        pdl_wait();                                    // the output may still be read by the kernel before
        uint32_t tile_it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, tile_it++) {
            int tp, tq, sp; decode(item, tp, tq, sp);
            const int a = tile_it & 1; const uint32_t aph = (tile_it >> 1) & 1;
            // the decision must be the same in every lane: tcgen05.ld is a warp-wide instruction
            const bool mine = !*abort_flag && mbar_wait(&acc_full[a], aph);
            if (!__all_sync(0xffffffffu, mine)) { ok = false; break; }
            tc_fence_after();
            const int prow = tp * BM + quarter * 32 + lane;            // row of P this thread holds
            const uint32_t t_addr = tmem_base + a * C::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
            for (int c0 = turn * CH; c0 < BN; c0 += (EPI_WARPS / 4) * CH) {
                uint32_t r[CH];
                if (CH == 32) tmem_ld32(t_addr + c0, r); else tmem_ld16(t_addr + c0, r);
                tmem_ld_wait();
                const int q0 = tq * BN + c0;                           // first row of Q in this chunk
                if constexpr (!SWAP) {
                    store_token_major<TOut, GATED, CH>(r, prow, q0, sp, p);
                } else if (GATED && SWAP) {
                    // Lanes 0..15 hold gates, lanes 16..31 the ups of the same 16 features.  Two tokens a round: the
                    // lower lanes hand over their gates of the second token and get the ups of the first, so that each
                    // half of the warp computes and stores one token.
                    const bool low = lane < 16;
                    const int feat = ((prow >> 5) << 4) + (lane & 15);
#pragma unroll
                    for (int j = 0; j < CH; j += 2) {
                        const float got = __shfl_xor_sync(0xffffffffu, __uint_as_float(low ? r[j + 1] : r[j]), 16);
                        const float g = low ? __uint_as_float(r[j]) : got;
                        const float u = low ? got : __uint_as_float(r[j + 1]);
                        const int tok = q0 + j + (low ? 0 : 1);
                        if (tok < p.rows_q && prow < p.rows_p)
                            ((bf16*)p.out)[(size_t)tok * p.ld_out + feat] = __float2bfloat16_rn(gated(g, u, p.act));
                    }
                } else {
                    // weight rows on lanes (prow), tokens on columns (q0 + j): lanes write neighbours
                    if (prow < p.rows_p) {
#pragma unroll
                        for (int j = 0; j < CH; j++) {
                            const int tok = q0 + j;
                            if (tok >= p.rows_q) break;
                            float v = __uint_as_float(r[j]);
                            if (p.splits > 1) {
                                p.partial[((size_t)sp * p.rows_q + tok) * p.rows_p + prow] = v;
                            } else {
                                if (p.cap > 0.f) v = softcap_f(v, p.cap);
                                ((TOut*)p.out)[(size_t)tok * p.ld_out + prow] = from_f<TOut>(v);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[a]);
        }
        if (!ok && !*abort_flag && lane == 0) { atomicExch(&g_gemm_error, 3); *abort_flag = 1; }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------
// The same product for many tokens on a pair of SMs (cta_group::2): a cluster of two CTAs owns a tile of 256 tokens
// by 256 weight rows.  Each CTA copies its 128 tokens of A and its 128 of the tile's weight rows into its own shared
// memory; one thread of the even CTA issues MMAs of 256 x 256 x 16 that read A and half of B from each CTA and leave
// each CTA's 128 tokens of the result in its own tensor memory.  A k-block of 64 then costs an SM 32 KB of shared
// memory and of copies instead of 48 KB: on one SM a 128 x 256 tile reads and refills its operands faster than the
// shared memory delivers them, which is what bounds the single-CTA kernel above.
//
// Barriers: both CTAs' copies count their bytes on the leader's `full` barrier (the leader expects both shares);
// a commit arrives on `empty` and `acc_full` at the same offset in both CTAs; the epilogue warps of both CTAs arrive
// on the leader's `acc_empty`.  All waits on these are bounded as above.  The two cluster barriers (after set-up,
// before the tensor memory is given back) are not: every path reaches them, since every loop before them ends.
// ---------------------------------------------------------------------------
struct PairCfg {
    static constexpr int BN = 256, HALF = 128;
    static constexpr int STAGE_BYTES = BM * BK * 2 + HALF * BK * 2;       // per CTA
    static constexpr int STAGES = (227 * 1024 - 1024 - 256) / STAGE_BYTES;   // 7: all of an SM's shared memory
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
};

template <typename TOut, bool GATED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, GemmParams p) {
    pdl_launch_dependents();
    using C = PairCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* full = bars;                       // [STAGES], the leader's is used
    uint64_t* empty = bars + C::STAGES;          // [STAGES], each CTA's own
    uint64_t* acc_full = bars + 2 * C::STAGES;   // [2], each CTA's own
    uint64_t* acc_empty = acc_full + 2;          // [2], the leader's is used
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();     // 0: the leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (threadIdx.x == 32) { tma_prefetch_map(&map_p); tma_prefetch_map(&map_q); }
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; a++) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 2 * EPI_WARPS); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
    tc_fence_before();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_items = p.tiles_p * p.tiles_q * p.splits;
    auto decode = [&](int item, int& tp, int& tq, int& sp) {
        sp = item % p.splits; item /= p.splits;
        tp = item % p.tiles_p; tq = item / p.tiles_p;
    };
    constexpr int A_OFF = 0, W_OFF = BM * BK * 2;

    if (warp == 0) {
        // ---------------- TMA producer, in both CTAs ----------------
        if (lane == 0) {
            const uint32_t lead_full = cluster_addr(&full[0], 0);
            uint32_t it = 0;
            bool ok = true, waited = false;
            for (int item = pair; item < n_items && ok; item += n_pairs) {
                int tp, tq, sp; decode(item, tp, tq, sp);
                const int kb0 = sp * p.kb_per_split, kb1 = min(p.kblocks, kb0 + p.kb_per_split);
                const int a_row = tp * 256 + (int)rank * BM, w_row = tq * C::BN + (int)rank * C::HALF;
                int kb = kb0;
                if (!waited) {
                    // weights first, then the wait for the kernel before this one, then its output
                    const int pre = min(kb1 - kb0, C::STAGES);
                    for (int j = 0; j < pre; j++) {
                        if (rank == 0) mbar_expect_tx(&full[j], 2 * C::STAGE_BYTES);
                        tma_load_2d_pair(smem + j * C::STAGE_BYTES + W_OFF, &map_q, lead_full + 8 * j, (kb0 + j) * BK, w_row);
                    }
                    pdl_wait();
                    waited = true;
                    for (int j = 0; j < pre; j++)
                        tma_load_2d_pair(smem + j * C::STAGE_BYTES + A_OFF, &map_p, lead_full + 8 * j, (kb0 + j) * BK, a_row);
                    it = pre; kb = kb0 + pre;
                }
                for (; kb < kb1; kb++, it++) {
                    const int s = it % C::STAGES; const uint32_t ph = (it / C::STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) { ok = false; break; }
                    uint8_t* st = smem + s * C::STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * C::STAGE_BYTES);
                    tma_load_2d_pair(st + W_OFF, &map_q, lead_full + 8 * s, kb * BK, w_row);
                    tma_load_2d_pair(st + A_OFF, &map_p, lead_full + 8 * s, kb * BK, a_row);
                }
            }
            if (!ok) {
                if (!*abort_flag) { atomicExch(&g_gemm_error, 4); *abort_flag = 1; }
                // the leader's barriers count both CTAs' copies: wait for those already issued
                if (rank == 0)
                    for (uint32_t back = 1; back <= (uint32_t)C::STAGES && back <= it; back++) {
                        const uint32_t j = it - back;
                        mbar_wait(&full[j % C::STAGES], (j / C::STAGES) & 1);
                    }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer, in the leader ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc_pair(C::BN);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int item = pair; item < n_items && ok; item += n_pairs, tile_it++) {
                int tp, tq, sp; decode(item, tp, tq, sp);
                const int kb0 = sp * p.kb_per_split, kb1 = min(p.kblocks, kb0 + p.kb_per_split);
                const int a = tile_it & 1; const uint32_t aph = (tile_it >> 1) & 1;
                if (*abort_flag || !mbar_wait(&acc_empty[a], aph ^ 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_addr = tmem_base + a * C::BN;
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % C::STAGES; const uint32_t ph = (it / C::STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&full[s], ph)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
                    const uint32_t sb = sa + W_OFF;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        umma_bf16_pair(d_addr, smem_desc(sa + k * UMMA_K * 2), smem_desc(sb + k * UMMA_K * 2), idesc,
                                       (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty[s]);           // frees the stage in both CTAs
                }
                if (ok) umma_commit_pair(&acc_full[a]);    // the accumulator is complete in both CTAs
            }
            if (!ok && !*abort_flag) { atomicExch(&g_gemm_error, 5); *abort_flag = 1; }
        }
    } else {
        // ---------------- epilogue: warps 2..9 of both CTAs ----------------
        const int quarter = warp & 3;
        const int turn = (warp - 2) >> 2;
        const uint32_t lead_acc_empty = cluster_addr(&acc_empty[0], 0);
        pdl_wait();
        uint32_t tile_it = 0;
        bool ok = true;
        for (int item = pair; item < n_items && ok; item += n_pairs, tile_it++) {
            int tp, tq, sp; decode(item, tp, tq, sp);
            const int a = tile_it & 1; const uint32_t aph = (tile_it >> 1) & 1;
            const bool mine = !*abort_flag && mbar_wait(&acc_full[a], aph);
            if (!__all_sync(0xffffffffu, mine)) { ok = false; break; }
            tc_fence_after();
            const int prow = tp * 256 + (int)rank * BM + quarter * 32 + lane;
            const uint32_t t_addr = tmem_base + a * C::BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = turn * 32; c0 < C::BN; c0 += (EPI_WARPS / 4) * 32) {
                uint32_t r[32];
                tmem_ld32(t_addr + c0, r);
                tmem_ld_wait();
                store_token_major<TOut, GATED, 32>(r, prow, tq * C::BN + c0, sp, p);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_acc_empty + 8 * a);
        }
        if (!ok && !*abort_flag && lane == 0) { atomicExch(&g_gemm_error, 6); *abort_flag = 1; }
    }

    tc_fence_before();
    cluster_sync();
    tc_fence_after();
    if (warp == 1) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
}

// partial[splits][rows][cols] summed in split order, then cap and conversion.
template <typename TOut>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TOut* __restrict__ out, int rows, int cols,
                                     long long ld_out, int splits, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t n = (size_t)rows * cols;
    if (i >= n) return;
    float s = 0.f;
    for (int k = 0; k < splits; k++) s += partial[(size_t)k * n + i];
    if (cap > 0.f) s = softcap_f(s, cap);
    out[(i / cols) * ld_out + (i % cols)] = from_f<TOut>(s);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
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

// rows x K bf16 matrix with row stride ld (elements); box = box_rows x 64 elements, 128-byte swizzle.
static int make_map(CUtensorMap* m, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return tb_refuse("gemm_tc: the driver does not provide cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return tb_refuse("gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

static int g_sms = 0;

template <int BN, bool SWAP, typename TOut, bool GATED = false, bool WIDE = false>
static int launch(const CUtensorMap& mp, const CUtensorMap& mq, const GemmParams& p, cudaStream_t stream) {
    using C = Cfg<BN, SWAP, WIDE>;
    static bool attr_set = false;
    auto kern = gemm_tc_kernel<BN, SWAP, TOut, GATED, WIDE>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int items = p.tiles_p * p.tiles_q * p.splits;
    const int grid = items < g_sms ? items : g_sms;
    tb_launch(kern, dim3(grid), dim3(GEMM_THREADS), C::SMEM, stream, mp, mq, p);
    return tb_launch_status();
}

// Many-token products on pairs of SMs: 0 never, 1 whenever the shape allows, 2 where it pays.  The environment
// variable TRAPETUM_GEMM_PAIR sets the start value (for profiling one kernel on every shape).
static int pair_policy_from_env() {
    const char* e = getenv("TRAPETUM_GEMM_PAIR");
    return (e && e[0] >= '0' && e[0] <= '2' && !e[1]) ? e[0] - '0' : 2;
}
static int g_pair = pair_policy_from_env();
static int g_pair_clusters = 0;

// Sets that policy (for comparisons and tests); returns the previous setting.
extern "C" int tb_gemm_tc_set_pair(int mode) { const int was = g_pair; g_pair = mode < 0 ? 0 : mode > 2 ? 2 : mode; return was; }

// Where the pair kernel pays.  Its launch costs about a microsecond more (a cluster is placed, two cluster barriers),
// its main loop runs 5 to 10 % faster.  Measured against the single-SM kernel with weights from memory, 512 to 8,192
// tokens on the 2B, 9B and 27B shapes: from about 300 k-blocks of work per pair on the pair is 3 to 12 % faster;
// below, equal or up to 7 % slower.  Whole prompts under sustained load (blocks of twelve repetitions, alternating):
// 27B shape at 2,048 tokens 98.8 -> 95.0 ms, 2B shape at 8,192 tokens 42.2 -> 41.3 ms, 9B shape at 2,048 equal; the 2B
// shape at 2,048 tokens has no product that long and does not use it.
static bool pair_pays(int M, int N, int K) {
    const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    const long long kblocks = (K + BK - 1) / BK;
    return tiles * kblocks >= 300LL * (g_sms / 2);
}

template <typename TOut, bool GATED>
static int launch_pair(const CUtensorMap& mp, const CUtensorMap& mq, const GemmParams& p, cudaStream_t stream) {
    using C = PairCfg;
    static bool attr_set = false;
    auto kern = gemm_tc_pair_kernel<TOut, GATED>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    if (!g_pair_clusters) {
        // how many pairs the device runs at once (an SM without a free neighbour takes none)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (g_sms / 2)); cfg.blockDim = dim3(GEMM_THREADS); cfg.dynamicSmemBytes = C::SMEM;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = g_sms / 2; }
        g_pair_clusters = n < g_sms / 2 ? n : g_sms / 2;
    }
    const int items = p.tiles_p * p.tiles_q * p.splits;
    const int pairs = items < g_pair_clusters ? items : g_pair_clusters;
    tb_launch(kern, dim3(2 * pairs), dim3(GEMM_THREADS), C::SMEM, stream, mp, mq, p);
    return tb_launch_status();
}

extern "C" int tb_gemm_tc_takes(const void* A, const void* W, int M, int N, int K, long long lda, long long ldw) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8 || lda % 8 || ldw % 8) return 0;
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 0;
    return 1;
}

extern "C" long long tb_gemm_tc_scratch_floats(int M, int N, int splits) {
    return splits > 1 ? (long long)splits * M * N : 0;
}

// How many K splits a small-token product should use so that about one CTA per SM streams weights.
extern "C" int tb_gemm_tc_splits(int M, int N, int K, int sms) {
    if (M > BM) return 1;
    const int tiles = (N + BM - 1) / BM;
    const int kblocks = (K + BK - 1) / BK;
    if (tiles * 2 > sms) return 1;
    int s = sms / tiles;
    if (s > kblocks / 2) s = kblocks / 2;          // at least two k-blocks per split
    if (s > 16) s = 16;
    if (s < 1) s = 1;
    const int per = (kblocks + s - 1) / s;
    return (kblocks + per - 1) / per;              // every split non-empty
}

// The split count a call really uses: every split gets the same number of k-blocks and none is empty.
extern "C" int tb_gemm_tc_effective_splits(int K, int splits) {
    const int kblocks = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > kblocks) splits = kblocks;
    const int per = (kblocks + splits - 1) / splits;
    return (kblocks + per - 1) / per;
}

// reduce = 0 with splits > 1: leave the partial sums in `scratch` ([splits][M][N]) for the consumer to add.
extern "C" int tb_gemm_tc(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K,
                          long long lda, long long ldw, long long ldc, float softcap, int splits, float* scratch,
                          int reduce, int gated_act, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!tb_gemm_tc_takes(A, W, M, N, K, lda, ldw))
        return tb_refuse("gemm_tc: needs K, lda, ldw multiples of 8 and 16-byte aligned operands "
                         "(M=%d N=%d K=%d lda=%lld ldw=%lld)", M, N, K, lda, ldw);
    if (c_dtype != TB_F32 && c_dtype != TB_BF16) return tb_refuse("gemm_tc: unknown output dtype %d", c_dtype);
    if (!g_sms) {
        int dev = 0; cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_sms <= 0) g_sms = 148;
    }
    const int kblocks = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > kblocks) splits = kblocks;
    int per = (kblocks + splits - 1) / splits;
    splits = (kblocks + per - 1) / per;
    if (splits > 1 && scratch == nullptr) return tb_refuse("gemm_tc: split-K needs scratch");
    const bool gated = gated_act >= 0;
    if (gated) {
        if (gated_act > 1) return tb_refuse("gemm_tc: unknown gated activation %d", gated_act);
        if (N % 32) return tb_refuse("gemm_tc: the gated epilogue needs a multiple of 32 weight rows, got %d", N);
        if (c_dtype != TB_BF16) return tb_refuse("gemm_tc: the gated epilogue writes bfloat16");
        if (softcap > 0.f) return tb_refuse("gemm_tc: the gated epilogue takes no soft cap");
        splits = 1; per = kblocks;                   // the activation is not linear: no partial sums
    }

    const bool swap = M <= BM;
    const bool pair = !swap && N >= 256 && (g_pair == 1 || (g_pair == 2 && pair_pays(M, N, K)));
    const bool wide = (long long)N * K * 2 >= (long long)TB_WIDE_FROM_BYTES;
    int bn;
    if (swap) bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    else bn = N >= 256 ? 256 : 128;

    GemmParams p;
    p.K = K; p.kblocks = kblocks; p.splits = splits; p.kb_per_split = per;
    p.out = C; p.ld_out = ldc; p.partial = scratch; p.cap = splits > 1 ? 0.f : softcap;
    p.act = gated ? gated_act : 0;
    CUtensorMap mp, mq;
    if (swap) {
        p.rows_p = N; p.rows_q = M;
        if (make_map(&mp, W, N, K, ldw, BM) || make_map(&mq, A, M, K, lda, bn)) return -1;
    } else {
        p.rows_p = M; p.rows_q = N;
        if (make_map(&mp, A, M, K, lda, BM) || make_map(&mq, W, N, K, ldw, pair ? PairCfg::HALF : bn)) return -1;
    }
    p.tiles_p = (p.rows_p + (pair ? 256 : BM) - 1) / (pair ? 256 : BM);
    p.tiles_q = (p.rows_q + bn - 1) / bn;

    int st;
#define GO(BN_, SW_) (c_dtype == TB_BF16 ? launch<BN_, SW_, bf16>(mp, mq, p, stream) : launch<BN_, SW_, float>(mp, mq, p, stream))
    if (gated) {
#define GG(BN_, SW_) launch<BN_, SW_, bf16, true>(mp, mq, p, stream)
        if (swap) st = bn == 16 ? (wide ? launch<16, true, bf16, true, true>(mp, mq, p, stream) : GG(16, true))
                     : bn == 32 ? GG(32, true) : bn == 64 ? GG(64, true) : GG(128, true);
        else if (pair) st = launch_pair<bf16, true>(mp, mq, p, stream);
        else st = bn == 256 ? GG(256, false) : GG(128, false);
#undef GG
    } else if (swap) {
        switch (bn) {
        case 16:
            // a long stream of weights: the kernel's own bytes in flight count for more than the overlap with its
            // neighbours, so it takes the whole SM
            if (c_dtype == TB_F32 && wide) st = launch<16, true, float, false, true>(mp, mq, p, stream);
            else st = GO(16, true);
            break;
        case 32: st = GO(32, true); break;
        case 64: st = GO(64, true); break;
        default: st = GO(128, true); break;
        }
    } else if (pair) {
        st = c_dtype == TB_BF16 ? launch_pair<bf16, false>(mp, mq, p, stream) : launch_pair<float, false>(mp, mq, p, stream);
    } else {
        st = bn == 256 ? GO(256, false) : GO(128, false);
    }
#undef GO
    if (st) return st;
    if (splits > 1 && reduce) {
        const size_t n = (size_t)M * N;
        const unsigned blocks = (unsigned)((n + 255) / 256);
        if (c_dtype == TB_BF16)
            tb_launch(splitk_reduce_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, scratch, (bf16*)C, M, N, ldc, splits, softcap);
        else
            tb_launch(splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream, scratch, (float*)C, M, N, ldc, splits, softcap);
        st = tb_launch_status();
    }
    return st;
}

// out[rows][cols] = sum over splits, in order, of partial[s][rows][cols] (32-bit).
extern "C" int tb_sum_partials(const float* partial, float* out, int rows, int cols, int splits, cudaStream_t stream) {
    const size_t n = (size_t)rows * cols;
    if (n == 0) return 0;
    if (splits < 1) return tb_refuse("sum_partials: splits=%d", splits);
    tb_launch(splitk_reduce_kernel<float>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
              partial, out, rows, cols, (long long)cols, splits, 0.f);
    return tb_launch_status();
}

// Reads and clears the error word (0 = no wait ran out).  Synchronises the device.
extern "C" int tb_gemm_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

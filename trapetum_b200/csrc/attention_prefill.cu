// Prefill attention on tensor cores (bfloat16): causal, packed sequences of unequal length,
// optional sliding window and tanh soft cap, grouped-query heads.
//
// The reference has no prefill kernel: a prompt goes through its one-query attn_k once per
// token (runtime/src/bin/gemma_run.rs:12; runtime/cuda/codebook_gemv.cu:240-270).  The formula
// is that kernel's: s = q.k * scale, s = cap*tanh(s/cap), softmax with the running maximum
// subtracted, sum of p*v; all of it in 32-bit except the two matrix products, which take
// bfloat16 operands (p is rounded to bfloat16 for p*v) and accumulate in 32-bit.
//
// One CTA = 64 queries of one head of one sequence (4 warps x 16 rows); keys and values stream
// through shared memory in tiles of 64 (32 for head sizes above 128) with cp.async double buffering; Q.K^T and P.V are
// mma.sync m16n8k16; the running softmax lives in registers (two rows per lane).  Rows of shared
// memory are padded by 16 bytes, which makes every ldmatrix conflict-free for any head_dim that
// is a multiple of 16.  Key tiles wholly outside a query block's causal/window range are skipped.
//
// This file is compiled once per head size (-DTB_HD=<head_dim>), head_dim % 16 == 0, <= 256.
#include "common.cuh"

TB_EXPORT_ERROR()

#ifndef TB_HD
#define TB_HD 256
#endif

#define BM 64
#define NWARPS 4
constexpr int HD = TB_HD;
constexpr int BN = HD > 128 ? 32 : 64;           // keys per tile: two CTAs fit on an SM at every head size
constexpr int PITCH = HD * 2 + 16;               // bytes per shared-memory row
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head_dim must be a multiple of 16, at most 256");

struct PrefillArgs {
    const bf16* q; const bf16* k; const bf16* v;
    long long q_stride, kv_stride;                // elements between token rows
    const int* seq_start;                         // [B + 1]
    bf16* out;                                    // [T, n_heads * HD]
    int n_heads, n_kv_heads, window;
    float scale, cap;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                 // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&h;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// cap * tanh(x / cap) as cap - 2 cap / (2^(x * c2) + 1) with c2 = 2 log2(e) / cap: two special-function
// instructions, absolute error of tanh about 1e-7 (the exponent is clamped so that 2^. stays finite)
__device__ __forceinline__ float softcap_fast(float x, float c2, float cap) {
    const float e = ex2(fminf(fmaxf(x * c2, -40.f), 40.f));
    return fmaf(-2.f * cap, rcp(e + 1.f), cap);
}

// rows [row0, row0 + ROWS) of a token-major matrix (row stride in elements) -> padded shared rows;
// rows at or beyond row_end are zero-filled
template <int ROWS>
__device__ __forceinline__ void load_tile(uint8_t* dst, const bf16* src, long long stride, int row0, int row_end) {
    constexpr int CPR = HD / 8;                    // 16-byte chunks per row
    for (int c = threadIdx.x; c < ROWS * CPR; c += NWARPS * 32) {
        const int r = c / CPR, ch = c % CPR;
        const bool valid = row0 + r < row_end;
        const bf16* s = src + (size_t)(valid ? row0 + r : row0) * stride + ch * 8;
        cp_async16(dst + r * PITCH + ch * 16, s, valid);
    }
}

__global__ void __launch_bounds__(NWARPS * 32) attn_prefill_mma_kernel(PrefillArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;                                   // [BM][PITCH]
    uint8_t* sK = sQ + BM * PITCH;                        // [2][BN][PITCH]
    uint8_t* sV = sK + 2 * BN * PITCH;                    // [2][BN][PITCH]

    const int b = blockIdx.z, h = blockIdx.y;
    const int s0 = a.seq_start[b], len = a.seq_start[b + 1] - s0;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;  // the blocks with most keys start first
    const int m0 = qb * BM;
    if (m0 >= len) return;
    const int kvh = h / (a.n_heads / a.n_kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const bf16* qbase = a.q + (size_t)s0 * a.q_stride + (size_t)h * HD;
    const bf16* kbase = a.k + (size_t)s0 * a.kv_stride + (size_t)kvh * HD;
    const bf16* vbase = a.v + (size_t)s0 * a.kv_stride + (size_t)kvh * HD;

    // keys this block can see: j <= i, i - j < window, over rows i in [m0, min(len, m0 + BM))
    const int i_last = min(len, m0 + BM) - 1;
    const int j_lo = (a.window > 0) ? max(0, m0 - a.window + 1) : 0;
    const int nb_lo = j_lo / BN, nb_hi = i_last / BN + 1;

    load_tile<BM>(sQ, qbase, a.q_stride, m0, len);
    load_tile<BN>(sK, kbase, a.kv_stride, nb_lo * BN, len);
    load_tile<BN>(sV, vbase, a.kv_stride, nb_lo * BN, len);
    cp_async_commit();

    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_a = m0 + warp * 16 + g, row_b = row_a + 8;       // the two query rows of this lane
    const float LOG2E = 1.4426950408889634f;
    const float cap_c2 = a.cap > 0.f ? 2.f * LOG2E / a.cap : 0.f;

    for (int nb = nb_lo; nb < nb_hi; nb++) {
        const int st = (nb - nb_lo) & 1;
        if (nb + 1 < nb_hi) {
            load_tile<BN>(sK + (st ^ 1) * BN * PITCH, kbase, a.kv_stride, (nb + 1) * BN, len);
            load_tile<BN>(sV + (st ^ 1) * BN * PITCH, vbase, a.kv_stride, (nb + 1) * BN, len);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint8_t* k_s = sK + st * BN * PITCH;
        const uint8_t* v_s = sV + st * BN * PITCH;

        // ---- S = Q K^T for this warp's 16 rows and the tile's 64 keys
        float s[BN / 8][4];
#pragma unroll
        for (int n = 0; n < BN / 8; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t qa[4];
            ldsm_x4(smem_addr(sQ + (warp * 16 + (lane & 15)) * PITCH + (ks * 16 + (lane >> 4) * 8) * 2), qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
            for (int n = 0; n < BN / 8; n += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_addr(k_s + (n * 8 + (lane >> 4) * 8 + (lane & 7)) * PITCH + (ks * 16 + ((lane >> 3) & 1) * 8) * 2),
                        b0, b1, b2, b3);
                mma_bf16(s[n], qa, b0, b1);
                mma_bf16(s[n + 1], qa, b2, b3);
            }
        }
        // ---- scale, cap, mask
        const int j0 = nb * BN;
        const bool edge = (j0 + BN - 1 > m0) || (j0 + BN > len) || (a.window > 0 && (m0 + BM - 1) - j0 >= a.window);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < BN / 8; n++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = s[n][e] * a.scale;
                if (a.cap > 0.f) v = softcap_fast(v, cap_c2, a.cap);
                if (edge) {
                    const int i = (e < 2) ? row_a : row_b;
                    const int j = j0 + n * 8 + 2 * t + (e & 1);
                    const bool vis = j <= i && j < len && (a.window <= 0 || i - j < a.window);
                    if (!vis) v = -INFINITY;
                }
                s[n][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        // ---- running softmax (rows are spread over the 4 lanes of a quad)
        float corr[2], msafe[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(m_run[r], mx[r]);
            msafe[r] = (mn == -INFINITY) ? 0.f : mn;
            corr[r] = (m_run[r] == -INFINITY) ? 0.f : ex2((m_run[r] - msafe[r]) * LOG2E);
            m_run[r] = mn;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int d = 0; d < HD / 8; d++) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
        uint32_t pa[BN / 16][4];
#pragma unroll
        for (int n = 0; n < BN / 8; n++) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                p[e] = ex2((s[n][e] - msafe[e >> 1]) * LOG2E);        // 2^(-inf) = 0 for masked keys
                l_run[e >> 1] += p[e];
            }
            pa[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; kk++) {
#pragma unroll
            for (int d = 0; d < HD / 8; d += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(smem_addr(v_s + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PITCH + (d * 8 + (lane >> 4) * 8) * 2),
                          b0, b1, b2, b3);
                mma_bf16(o[d], pa[kk], b0, b1);
                mma_bf16(o[d + 1], pa[kk], b2, b3);
            }
        }
        __syncthreads();                           // the next iteration's loads overwrite this stage's partner
    }

    // ---- finish: row sums over the quad, divide, store
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv_a = 1.f / l_run[0], inv_b = 1.f / l_run[1];
    bf16* orow_a = a.out + ((size_t)(s0 + row_a) * a.n_heads + h) * HD;
    bf16* orow_b = a.out + ((size_t)(s0 + row_b) * a.n_heads + h) * HD;
#pragma unroll
    for (int d = 0; d < HD / 8; d++) {
        if (row_a < len) *(uint32_t*)(orow_a + d * 8 + 2 * t) = pack_bf16(o[d][0] * inv_a, o[d][1] * inv_a);
        if (row_b < len) *(uint32_t*)(orow_b + d * 8 + 2 * t) = pack_bf16(o[d][2] * inv_b, o[d][3] * inv_b);
    }
}

extern "C" int tb_attn_prefill_head_dim() { return HD; }

extern "C" int tb_attn_prefill_mma(const void* q, const void* k, const void* v, long long q_stride, long long kv_stride,
                                   const int* seq_start, void* out, int batch, int max_seq_len, int n_heads,
                                   int n_kv_heads, int hd, float scale, float cap, int window, cudaStream_t stream) {
    if (batch <= 0 || max_seq_len <= 0) return 0;
    if (hd != HD) return tb_refuse("attn_prefill: this library is built for head_dim %d, got %d", HD, hd);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads)
        return tb_refuse("attn_prefill: %d heads cannot share %d kv heads", n_heads, n_kv_heads);
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || (q_stride % 8) || (kv_stride % 8))
        return tb_refuse("attn_prefill: q, k, v rows must be 16-byte aligned");
    if (n_heads > 65535 || batch > 65535) return tb_refuse("attn_prefill: %d heads x %d sequences exceed one launch", n_heads, batch);
    PrefillArgs a;
    a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v;
    a.q_stride = q_stride; a.kv_stride = kv_stride; a.seq_start = seq_start; a.out = (bf16*)out;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.window = window; a.scale = scale; a.cap = cap;
    constexpr int SMEM = (BM + 4 * BN) * PITCH;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    dim3 grid((max_seq_len + BM - 1) / BM, n_heads, batch);
    tb_launch(attn_prefill_mma_kernel, dim3(grid), dim3(NWARPS * 32), SMEM, stream, a);
    return tb_launch_status();
}

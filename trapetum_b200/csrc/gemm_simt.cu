// C[M,N] = A[M,K] * W[N,K]^T on the 32-bit FMA pipe.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no
// reduced-precision matrix mode) and the any-size fallback of the bfloat16 path
// (sizes the tensor-core kernel refuses: K not a multiple of 8 elements, or
// 32-bit weights).  Weights are [out, in] as the checkpoint stores them, so a
// row of W is one output column's dot-product vector, like the reference's
// dense GEMV (runtime/cuda/codebook_gemv.cu:482-517).  Products and sums are
// 32-bit; each C element adds its K terms in the same order whatever M and N are
// (k-tiles of 16 in ascending order, each tile summed on its own first), so a
// token's result does not depend on what else is in the batch.
// Optional epilogue: tanh soft cap (the final logit cap, runtime/src/lib.rs:4559-4560).
#include "common.cuh"

TB_EXPORT_ERROR()

#define BM 64
#define BN 64
#define BK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C,
                 int M, int N, int K, long long lda, long long ldw, long long ldc, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = tid / 16, tc = tid % 16;          // 16x16 threads, 4x4 outputs each
    const int lr = tid / 4, lk = (tid % 4) * 4;      // loader: row lr, k offset lk..lk+3
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            const int m = m0 + lr, n = n0 + lr;
            As[lk + j][lr] = (m < M && k < K) ? to_f<TA>(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk + j][lr] = (n < N && k < K) ? to_f<TW>(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
        // blocked summation: the 16 products of a k-tile are added up on their own and the tile's sum is then
        // added to the running total, so that rounding errors grow with K/16 + 16 terms instead of K
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) part[i][j] = 0.f;
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][tr * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[k][tc * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) part[i][j] = fmaf(a[i], w[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + tr * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tc * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (cap > 0.f) v = softcap_f(v, cap);
            C[(size_t)m * ldc + n] = from_f<TC>(v);
        }
    }
}

extern "C" int tb_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                            int M, int N, int K, long long lda, long long ldw, long long ldc,
                            float softcap, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return tb_refuse("gemm: K=%d", K);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return tb_refuse("gemm: M=%d is too many rows for one call", M);
    const int key = (a_dtype << 2) | (w_dtype << 1) | c_dtype;
#define LAUNCH(TA, TW, TC) tb_launch(gemm_simt_kernel<TA, TW, TC>, dim3(grid), dim3(256), 0, stream,  \
        (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc, softcap)
    switch (key) {
    case 0: LAUNCH(float, float, float); break;
    case 1: LAUNCH(float, float, bf16); break;
    case 2: LAUNCH(float, bf16, float); break;
    case 3: LAUNCH(float, bf16, bf16); break;
    case 4: LAUNCH(bf16, float, float); break;
    case 5: LAUNCH(bf16, float, bf16); break;
    case 6: LAUNCH(bf16, bf16, float); break;
    case 7: LAUNCH(bf16, bf16, bf16); break;
    default: return tb_refuse("gemm: unknown dtype codes %d %d %d", a_dtype, w_dtype, c_dtype);
    }
#undef LAUNCH
    return tb_launch_status();
}

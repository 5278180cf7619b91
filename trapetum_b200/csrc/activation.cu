// Gated activation of the feed-forward: out = act(gate) * up.
//
// gelu_tanh(g) = 0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3))), the form the
// reference computes in gelu_mul_k (runtime/cuda/codebook_gemv.cu:531-537); silu
// is there for arrangements that want it (codebook_gemv.cu:205-209).  The input
// holds gate in columns [0, I) and up in [I, 2I) of each row; all math is 32-bit.
#include "common.cuh"

TB_EXPORT_ERROR()

#define ACT_GELU_TANH 0
#define ACT_SILU 1

__device__ __forceinline__ float gelu_tanh_f(float g) {
    return 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
}
__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

template <typename TI, typename TO, int ACT>
__global__ void gated_act_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int inter) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const float g = to_f<TI>(gu[row * 2 * inter + c]);
    const float u = to_f<TI>(gu[row * 2 * inter + inter + c]);
    const float a = (ACT == ACT_GELU_TANH) ? gelu_tanh_f(g) : silu_f(g);
    out[row * inter + c] = from_f<TO>(a * u);
}

extern "C" int tb_gated_act(const void* gu, int in_dtype, void* out, int out_dtype, int rows, int inter,
                            int act, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0) return tb_refuse("gated_act: intermediate size %d", inter);
    if (act != ACT_GELU_TANH && act != ACT_SILU) return tb_refuse("gated_act: unknown activation %d", act);
    dim3 grid(rows, (inter + 255) / 256);
    if (grid.y > 65535) return tb_refuse("gated_act: intermediate size %d is too wide", inter);
#define LAUNCH(TI, TO)                                                                         \
    do {                                                                                       \
        if (act == ACT_GELU_TANH) tb_launch(gated_act_kernel<TI, TO, ACT_GELU_TANH>, dim3(grid), dim3(256), 0, stream, (const TI*)gu, (TO*)out, inter); \
        else tb_launch(gated_act_kernel<TI, TO, ACT_SILU>, dim3(grid), dim3(256), 0, stream, (const TI*)gu, (TO*)out, inter);                       \
    } while (0)
    if (in_dtype == TB_F32 && out_dtype == TB_F32) LAUNCH(float, float);
    else if (in_dtype == TB_F32 && out_dtype == TB_BF16) LAUNCH(float, bf16);
    else if (in_dtype == TB_BF16 && out_dtype == TB_BF16) LAUNCH(bf16, bf16);
    else if (in_dtype == TB_BF16 && out_dtype == TB_F32) LAUNCH(bf16, float);
    else return tb_refuse("gated_act: unknown dtype codes %d %d", in_dtype, out_dtype);
#undef LAUNCH
    return tb_launch_status();
}

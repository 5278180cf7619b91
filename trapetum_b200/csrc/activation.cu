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

// x[r, c] += bias[c] in place, the sum in 32-bit (rows may be wider than `width`: row_stride elements apart).
template <typename T, typename TB>
__global__ void add_bias_kernel(T* __restrict__ x, long long row_stride, const TB* __restrict__ bias, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    T* p = x + (size_t)blockIdx.x * row_stride + c;
    *p = from_f<T>(to_f<T>(*p) + to_f<TB>(bias[c]));
}

extern "C" int tb_add_bias(void* x, int x_dtype, long long row_stride, const void* bias, int bias_dtype, int rows,
                           int width, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    dim3 grid(rows, (width + 255) / 256);
    if (grid.y > 65535) return tb_refuse("add_bias: width %d is too wide", width);
#define LAUNCH(T, TB) tb_launch(add_bias_kernel<T, TB>, dim3(grid), dim3(256), 0, stream, (T*)x, row_stride, (const TB*)bias, width)
    if (x_dtype == TB_F32 && bias_dtype == TB_F32) LAUNCH(float, float);
    else if (x_dtype == TB_F32 && bias_dtype == TB_BF16) LAUNCH(float, bf16);
    else if (x_dtype == TB_BF16 && bias_dtype == TB_BF16) LAUNCH(bf16, bf16);
    else if (x_dtype == TB_BF16 && bias_dtype == TB_F32) LAUNCH(bf16, float);
    else return tb_refuse("add_bias: unknown dtype codes %d %d", x_dtype, bias_dtype);
#undef LAUNCH
    return tb_launch_status();
}

// Shared helpers of the kernel files: dtype codes, conversions, warp and block
// reductions, and the error string that the Python side reads after a refusal.
//
// Every exported function is `extern "C" int tb_<name>(..., cudaStream_t)`:
// 0 = launched, >0 = a cudaError_t from the launch, <0 = the arguments were
// refused (tb_error() of the same library says why).  Nothing here allocates.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#define TB_F32 0
#define TB_BF16 1

static thread_local char tb_err_buf[512];

static int tb_refuse(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tb_err_buf, sizeof(tb_err_buf), fmt, ap);
    va_end(ap);
    return -1;
}

#define TB_EXPORT_ERROR()                                                     \
    extern "C" const char* tb_error() { return tb_err_buf; }

static inline int tb_launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  Every kernel of this library is launched with the attribute that
// lets it start while the kernel before it in the stream is still draining, begins with
// pdl_launch_dependents() (so that its own successor may be scheduled early too) and calls pdl_wait()
// before it first touches memory that an earlier kernel wrote or still reads.  pdl_wait() returns when
// the preceding kernel has completed and its writes are visible, so the order of effects is that of
// ordinary stream order; what overlaps is launch latency, block scheduling and whatever a kernel does
// before its wait (barrier set-up, tensor-memory allocation, loads of weights).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline void tb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);       // the status is read with tb_launch_status()
}

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions is fixed (lanes by xor tree, then warps by xor tree).
__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // red may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// tanh soft cap, `cap * tanh(x / cap)`, in 32-bit.
__device__ __forceinline__ float softcap_f(float x, float cap) { return cap * tanhf(x / cap); }

// Dispatch on a dtype code.
#define TB_DISPATCH_1(code, T, ...)                                           \
    do {                                                                      \
        if ((code) == TB_F32) { typedef float T; __VA_ARGS__; }               \
        else if ((code) == TB_BF16) { typedef bf16 T; __VA_ARGS__; }          \
        else return tb_refuse("unknown dtype code %d", (int)(code));          \
    } while (0)

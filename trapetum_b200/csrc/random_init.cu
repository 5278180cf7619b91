// Random weights made on the device: element i of a tensor is a function of (seed, tensor name, i) alone,
// so a model of any size is filled in place, tensor by tensor, with no host copy and in any order, and
// a model folder written on the host holds the same bits (weights/random_init.py is the numpy twin).
// The reference seeds an xorshift generator inside the program for its synthetic check models
// (runtime/src/lib.rs:1604-1629, runtime/src/bin/model.rs:158-177).
//
//   key      = FNV-1a-64(name) xor seed, as two 32-bit words (made on the host)
//   words    = Philox-4x32-10(counter = (i / 4, 0x54524150, 0), key)
//   normals  = Box-Muller on (words 0, 1) and on (words 2, 3): two numbers each
//   value    = bfloat16(normal * std), stored as bfloat16 or widened to float32
//
// Logarithm, sine and cosine are polynomials evaluated with round-to-nearest additions, multiplications
// and divisions only (the intrinsics below keep the compiler from fusing them), so that the host twin
// and the tests' plain version get the same bits.
#include "common.cuh"

TB_EXPORT_ERROR()

__device__ __forceinline__ void philox_4x32_10(uint32_t& c0, uint32_t& c1, uint32_t& c2, uint32_t& c3, uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
        const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
        c0 = n0; c1 = l1; c2 = n2; c3 = l0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}

// -ln(u) for u = ((w >> 8) + 1) / 2^24 in (0, 1]
__device__ __forceinline__ float neg_log_unit(uint32_t w) {
    const uint32_t k = (w >> 8) + 1u;
    const int e = 31 - __clz(k);
    const float m = __fmul_rn(__uint2float_rn(k), __int_as_float((127 - e) << 23));      // in [1, 2), exact
    const float s = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
    const float z = __fmul_rn(s, s);
    float p = 0.0909090936f;
    p = __fadd_rn(__fmul_rn(p, z), 0.111111112f);
    p = __fadd_rn(__fmul_rn(p, z), 0.142857149f);
    p = __fadd_rn(__fmul_rn(p, z), 0.200000003f);
    p = __fadd_rn(__fmul_rn(p, z), 0.333333343f);
    p = __fadd_rn(__fmul_rn(p, z), 1.0f);
    const float ln_m = __fmul_rn(2.0f, __fmul_rn(s, p));
    return __fsub_rn(__fmul_rn(__int2float_rn(24 - e), 0.693147182f), ln_m);
}

// (sin, cos) of 2 pi (w >> 6) / 2^26: the top two bits pick the quadrant, the next 24 the angle in it
__device__ __forceinline__ void sin_cos_turn(uint32_t w, float& sn, float& cs) {
    const float t = __fmul_rn(__fmul_rn(__uint2float_rn((w >> 6) & 0xFFFFFFu), 5.9604644775390625e-08f), 1.57079637f);
    const float z = __fmul_rn(t, t);
    float s = 1.60590444e-10f;
    s = __fadd_rn(__fmul_rn(s, z), -2.50521079e-08f);
    s = __fadd_rn(__fmul_rn(s, z), 2.75573188e-06f);
    s = __fadd_rn(__fmul_rn(s, z), -0.000198412701f);
    s = __fadd_rn(__fmul_rn(s, z), 0.00833333377f);
    s = __fadd_rn(__fmul_rn(s, z), -0.166666672f);
    s = __fmul_rn(__fadd_rn(__fmul_rn(s, z), 1.0f), t);
    float c = 2.08767559e-09f;
    c = __fadd_rn(__fmul_rn(c, z), -2.755732e-07f);
    c = __fadd_rn(__fmul_rn(c, z), 2.48015876e-05f);
    c = __fadd_rn(__fmul_rn(c, z), -0.00138888892f);
    c = __fadd_rn(__fmul_rn(c, z), 0.0416666679f);
    c = __fadd_rn(__fmul_rn(c, z), -0.5f);
    c = __fadd_rn(__fmul_rn(c, z), 1.0f);
    switch (w >> 30) {
    case 0: sn = s; cs = c; break;
    case 1: sn = c; cs = -s; break;
    case 2: sn = -s; cs = -c; break;
    default: sn = -c; cs = s; break;
    }
}

template <typename T>
__global__ void random_normal_kernel(T* out, long long n, uint32_t k0, uint32_t k1, float std) {
    pdl_launch_dependents();
    const long long blocks = (n + 3) >> 2;
    for (long long blk = (long long)blockIdx.x * blockDim.x + threadIdx.x; blk < blocks; blk += (long long)gridDim.x * blockDim.x) {
        uint32_t c0 = (uint32_t)blk, c1 = (uint32_t)((unsigned long long)blk >> 32), c2 = 0x54524150u, c3 = 0u;
        philox_4x32_10(c0, c1, c2, c3, k0, k1);
        float v[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t a = h ? c2 : c0, b = h ? c3 : c1;
            const float r = __fsqrt_rn(__fmul_rn(2.0f, neg_log_unit(a)));
            float sn, cs;
            sin_cos_turn(b, sn, cs);
            v[2 * h] = __fmul_rn(__fmul_rn(r, cs), std);
            v[2 * h + 1] = __fmul_rn(__fmul_rn(r, sn), std);
        }
        const long long i0 = blk << 2;
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (i0 + e < n) out[i0 + e] = from_f<T>(__bfloat162float(__float2bfloat16_rn(v[e])));
    }
}

// out[i] = bfloat16(normal_i * std) for i in [0, n), as bfloat16 (dtype 1) or widened to float32 (dtype 0)
extern "C" int tb_random_normal(void* out, int dtype, long long n, unsigned int k0, unsigned int k1, float std,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(std >= 0.f)) return tb_refuse("random_normal: std=%g must not be negative", (double)std);
    const long long blocks = (n + 3) >> 2;
    long long grid = (blocks + 255) / 256;
    if (grid > 148 * 32) grid = 148 * 32;
    TB_DISPATCH_1(dtype, T, tb_launch(random_normal_kernel<T>, dim3((unsigned)grid), dim3(256), 0, stream, (T*)out, n,
                                      (uint32_t)k0, (uint32_t)k1, std));
    return tb_launch_status();
}

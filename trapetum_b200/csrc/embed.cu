// Embedding lookup with scale, and row gather.
//
// embed: h[t, :] = float(E[id_t, :]) * scale, the product taken in 32-bit and
// stored in the 32-bit residual stream.  The reference bakes sqrt(hidden) into
// an fp16 table at export (model/export_gemma.py:59-61) and copies one row per
// token from the host (runtime/src/lib.rs:4555).  An id outside [0, vocab)
// yields a row of NaN, so that it cannot pass for a result.
#include "common.cuh"

TB_EXPORT_ERROR()

template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = __int_as_float(0x7fc00000);
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f<TW>(row[i]) * scale;
}

extern "C" int tb_embed(const int* ids, const void* table, int table_dtype, float* out,
                        int n_tokens, int hidden, int vocab, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return tb_refuse("embed: hidden=%d vocab=%d", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    TB_DISPATCH_1(table_dtype, TW,
        tb_launch(embed_kernel<TW>, dim3(n_tokens), dim3(threads), 0, stream, ids, (const TW*)table, out, hidden, vocab, scale));
    return tb_launch_status();
}

// out[i, :] = in[rows[i], :]; an index outside [0, n_rows) yields NaN.
__global__ void gather_rows_kernel(const float* __restrict__ in, const int* __restrict__ rows,
                                   float* __restrict__ out, int width, int n_rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int r = rows[i];
    float* o = out + (size_t)i * width;
    if (r < 0 || r >= n_rows) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = __int_as_float(0x7fc00000);
        return;
    }
    const float* s = in + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = s[c];
}

extern "C" int tb_gather_rows(const float* in, const int* rows, float* out, int n_out, int width,
                              int n_rows, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    tb_launch(gather_rows_kernel, dim3(n_out), dim3(256), 0, stream, in, rows, out, width, n_rows);
    return tb_launch_status();
}

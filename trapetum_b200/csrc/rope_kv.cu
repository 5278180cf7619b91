// Rotary position encoding of q and k, fused with the write of k and v into the
// paged cache.
//
// Rotation (rotate-half pairing, runtime/cuda/codebook_gemv.cu:219-230): for each
// head and i in [0, R/2), angle = pos * inv_freq[i];
//   (x[i], x[i+R/2]) <- (x[i] cos - x[i+R/2] sin,  x[i+R/2] cos + x[i] sin)
// with R = rotary_dim <= head_dim (dims >= R pass through).  Angle, sin and cos
// are 32-bit; the angle table inv_freq[i] = theta^(-2i/R) is made once by the
// position-encoding part.  The reference appends k and v to a flat per-layer
// cache with a device copy (codebook_gemv.cu:860-864); here rows go to pages:
//
//   row  = ring_rows ? pos % ring_rows : pos
//   page = page_table[seq, row / page_rows]
//   K[page, kv_head, row % page_rows, :] = k_rot      (V likewise, unrotated)
//
// The input may also be the split-K partial sums of the q/k/v product (32-bit): they are added in
// split order, rotated in 32-bit and rounded once.
//
// In a ring (a layer that only ever reads the last `window` keys) a prompt longer
// than the ring maps several tokens to one row; only tokens with
// pos >= len_after - ring_rows are written, so the newest one wins without a race.
#include "common.cuh"

TB_EXPORT_ERROR()

struct RopeKvArgs {
    void* qkv; long long row_stride;          // elements between token rows
    int q_off, k_off, v_off;                  // element offsets of q, k, v in a row
    int n_heads, n_kv_heads, head_dim, rotary_dim;
    const float* inv_freq;                    // [rotary_dim/2] or null: no rotation
    const int* positions;                     // [T]
    const int* token_seq;                     // [T] index of the token's sequence in the batch
    const int* len_after;                     // [B] tokens in cache after this step
    void* k_pool; void* v_pool;               // this cache line: [n_pages][n_kv][page_rows][head_dim]; null: no write
    const int* page_table; int pt_stride;     // [B, pt_stride]
    int page_rows; int ring_rows;
    const float* partial; int n_splits; long long split_stride, partial_row_stride;   // if set: the row's values are the sum over
                                                                  // splits of partial[s][t][col]; qkv is written
};

template <typename T>
__global__ void rope_kv_kernel(RopeKvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int hs = blockIdx.y;                      // head slot: q heads, then k heads, then v heads
    const int hd = a.head_dim, half = a.rotary_dim >> 1;
    T* row = (T*)a.qkv + (size_t)t * a.row_stride;
    const int pos = a.positions[t];
    const bool is_q = hs < a.n_heads;
    const bool is_k = !is_q && hs < a.n_heads + a.n_kv_heads;
    const int kvh = is_q ? 0 : (is_k ? hs - a.n_heads : hs - a.n_heads - a.n_kv_heads);
    const int col0 = is_q ? a.q_off + hs * hd : (is_k ? a.k_off + kvh * hd : a.v_off + kvh * hd);
    T* x = row + col0;
    // value of element i of this head: from the matrix itself, or summed from split-K partials (in split order)
    auto val = [&](int i) -> float {
        if (a.partial == nullptr) return to_f<T>(x[i]);
        const float* p = a.partial + (size_t)t * a.partial_row_stride + col0 + i;
        float v = p[0];
        for (int s = 1; s < a.n_splits; s++) v += p[(size_t)s * a.split_stride];
        return v;
    };
    const bool from_partial = a.partial != nullptr;

    T* dst = nullptr;
    if (!is_q && a.k_pool != nullptr) {
        const int b = a.token_seq[t];
        bool keep = true;
        int r = pos;
        if (a.ring_rows > 0) {
            keep = pos >= a.len_after[b] - a.ring_rows;
            r = pos % a.ring_rows;
        }
        if (keep) {
            const int page = a.page_table[(size_t)b * a.pt_stride + r / a.page_rows];
            T* pool = (T*)(is_k ? a.k_pool : a.v_pool);
            dst = pool + (((size_t)page * a.n_kv_heads + kvh) * a.page_rows + (r % a.page_rows)) * hd;
        }
    }

    if (!is_q && !is_k) {                            // v: copy only
        for (int i = threadIdx.x; i < hd; i += blockDim.x) {
            const T y = from_partial ? from_f<T>(val(i)) : x[i];
            if (from_partial) x[i] = y;
            if (dst) dst[i] = y;
        }
        return;
    }
    const bool rotate = a.inv_freq != nullptr;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        // each thread owns a pair (i, i+half) for i < half, or a pass-through dim
        if (rotate && i < half) {
            const float ang = (float)pos * a.inv_freq[i];
            float s, c;
            sincosf(ang, &s, &c);
            const float x0 = val(i), x1 = val(i + half);
            const T y0 = from_f<T>(x0 * c - x1 * s), y1 = from_f<T>(x1 * c + x0 * s);
            x[i] = y0; x[i + half] = y1;
            if (dst) { dst[i] = y0; dst[i + half] = y1; }
        } else if (!rotate || i >= 2 * half) {
            const T y = from_partial ? from_f<T>(val(i)) : x[i];
            if (from_partial) x[i] = y;
            if (dst) dst[i] = y;
        }
    }
}

extern "C" int tb_rope_kv(const RopeKvArgs* args, int dtype, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    RopeKvArgs a = *args;
    if (a.head_dim <= 0 || a.rotary_dim < 0 || a.rotary_dim > a.head_dim || (a.rotary_dim & 1))
        return tb_refuse("rope: head_dim=%d rotary_dim=%d (rotary_dim must be even and <= head_dim)",
                         a.head_dim, a.rotary_dim);
    if (a.k_pool != nullptr && (a.page_rows <= 0 || a.page_table == nullptr || a.v_pool == nullptr))
        return tb_refuse("rope: a cache write needs page_rows > 0, a page table and both pools");
    if (a.ring_rows > 0 && a.ring_rows % a.page_rows != 0)
        return tb_refuse("rope: ring_rows=%d must be a multiple of page_rows=%d", a.ring_rows, a.page_rows);
    const int slots = a.n_heads + 2 * a.n_kv_heads;
    int threads = 32;
    while (threads < 256 && threads < a.head_dim / 2) threads <<= 1;
    dim3 grid(n_tokens, slots);
    TB_DISPATCH_1(dtype, T, tb_launch(rope_kv_kernel<T>, dim3(grid), dim3(threads), 0, stream, a));
    return tb_launch_status();
}

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

// One CTA per token (several when tokens are few).  threadIdx.x walks the rotary pairs two at a time (4-byte accesses for bfloat16),
// threadIdx.y strides over the head slots (q heads, then k heads, then v heads), so the sine and cosine of
// a pair are computed once per thread and reused for every head it visits.
template <typename T>
__global__ void rope_kv_kernel(RopeKvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int hd = a.head_dim, half = a.rotary_dim >> 1;
    T* row = (T*)a.qkv + (size_t)t * a.row_stride;
    const int pos = a.positions[t];
    const bool rotate = a.inv_freq != nullptr && half > 0;
    const bool from_partial = a.partial != nullptr;
    const float* prow = from_partial ? a.partial + (size_t)t * a.partial_row_stride : nullptr;

    // where this token's k and v go in the cache (if anywhere)
    size_t cache_off = 0;
    bool store = false;
    if (a.k_pool != nullptr) {
        const int b = a.token_seq[t];
        store = true;
        int r = pos;
        if (a.ring_rows > 0) {
            store = pos >= a.len_after[b] - a.ring_rows;
            r = pos % a.ring_rows;
        }
        if (store) {
            const int page = a.page_table[(size_t)b * a.pt_stride + r / a.page_rows];
            cache_off = ((size_t)page * a.n_kv_heads * a.page_rows + (r % a.page_rows)) * hd;
        }
    }
    auto val = [&](int col) -> float {               // element `col` of the token's row
        if (!from_partial) return to_f<T>(row[col]);
        float v = prow[col];
        for (int s = 1; s < a.n_splits; s += 4) {    // loads of four splits at a time, then added in order
            float t4[4];
#pragma unroll
            for (int k = 0; k < 4; k++) t4[k] = (s + k < a.n_splits) ? prow[(size_t)(s + k) * a.split_stride + col] : 0.f;
#pragma unroll
            for (int k = 0; k < 4; k++) if (s + k < a.n_splits) v += t4[k];
        }
        return v;
    };

    const int i0 = threadIdx.x * 2;                  // this thread's pairs: i0 and i0 + 1
    float sn[2] = {0.f, 0.f}, cs[2] = {1.f, 1.f};
    if (rotate) {
#pragma unroll
        for (int e = 0; e < 2; e++)
            if (i0 + e < half) sincosf((float)pos * a.inv_freq[i0 + e], &sn[e], &cs[e]);
    }
    const int slots = a.n_heads + 2 * a.n_kv_heads;
    for (int hs = blockIdx.y * blockDim.y + threadIdx.y; hs < slots; hs += gridDim.y * blockDim.y) {
        const bool is_q = hs < a.n_heads;
        const bool is_k = !is_q && hs < a.n_heads + a.n_kv_heads;
        const int kvh = is_q ? 0 : (is_k ? hs - a.n_heads : hs - a.n_heads - a.n_kv_heads);
        const int col0 = is_q ? a.q_off + hs * hd : (is_k ? a.k_off + kvh * hd : a.v_off + kvh * hd);
        T* x = row + col0;
        T* dst = nullptr;
        if (!is_q && store)
            dst = (T*)(is_k ? a.k_pool : a.v_pool) + cache_off + (size_t)kvh * a.page_rows * hd;
        if ((is_q || is_k) && rotate) {
            // the thread's first two pairs use the sines and cosines made above; a head with more pairs than
            // the CTA has threads for (rotary_dim > 4 * blockDim.x) goes round again and makes its own
            for (int ib = i0; ib < half; ib += blockDim.x * 2) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int i = ib + e;
                    if (i < half) {
                        float sne = sn[e], cse = cs[e];
                        if (ib != i0) sincosf((float)pos * a.inv_freq[i], &sne, &cse);
                        const float x0 = val(col0 + i), x1 = val(col0 + i + half);
                        const T y0 = from_f<T>(x0 * cse - x1 * sne), y1 = from_f<T>(x1 * cse + x0 * sne);
                        x[i] = y0; x[i + half] = y1;
                        if (dst) { dst[i] = y0; dst[i + half] = y1; }
                    }
                }
            }
            // dims beyond the rotary part pass through
            for (int i = 2 * half + i0; i < hd; i += blockDim.x * 2)
#pragma unroll
                for (int e = 0; e < 2; e++) if (i + e < hd) {
                    const T y = from_partial ? from_f<T>(val(col0 + i + e)) : x[i + e];
                    if (from_partial) x[i + e] = y;
                    if (dst) dst[i + e] = y;
                }
        } else if (dst != nullptr || from_partial) {
            // v heads, or no rotation at all: copy (and round, when the source is partial sums)
            for (int i = i0; i < hd; i += blockDim.x * 2)
#pragma unroll
                for (int e = 0; e < 2; e++) if (i + e < hd) {
                    const T y = from_partial ? from_f<T>(val(col0 + i + e)) : x[i + e];
                    if (from_partial) x[i + e] = y;
                    if (dst) dst[i + e] = y;
                }
        }
    }
}

// The same for many tokens (a prompt), bfloat16, head_dim a multiple of 16 with the whole head rotated or
// rotary_dim a multiple of 16: one warp per token, 16-byte accesses.  A lane owns eight neighbouring pairs
// (dims i..i+7 and i+half..i+half+7) of every second head slot; their sines and cosines are computed once and
// reused for all the heads the lane visits.
__global__ void __launch_bounds__(256, 2) rope_kv_rows_kernel(RopeKvArgs a, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    const int hd = a.head_dim, half = a.rotary_dim >> 1;
    const int groups = half >> 3;                       // groups of eight pairs per head (0: no rotation)
    const int chunks = hd >> 3;                         // 16-byte chunks per head
    bf16* row = (bf16*)a.qkv + (size_t)t * a.row_stride;
    const int pos = a.positions[t];
    size_t cache_off = 0;
    bool store = false;
    if (a.k_pool != nullptr) {
        const int b = a.token_seq[t];
        store = true;
        int r = pos;
        if (a.ring_rows > 0) { store = pos >= a.len_after[b] - a.ring_rows; r = pos % a.ring_rows; }
        if (store) {
            const int page = a.page_table[(size_t)b * a.pt_stride + r / a.page_rows];
            cache_off = ((size_t)page * a.n_kv_heads * a.page_rows + (r % a.page_rows)) * hd;
        }
    }
    auto unpack = [](const uint4& w, float* f) {
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
    };
    auto pack = [](const float* f) -> uint4 {
        uint32_t u[4];
#pragma unroll
        for (int i = 0; i < 4; i++) { __nv_bfloat162 h2 = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); u[i] = *(uint32_t*)&h2; }
        return make_uint4(u[0], u[1], u[2], u[3]);
    };
    const int qk_slots = a.n_heads + a.n_kv_heads;
    // ---- what is only copied to the cache (k dims beyond the rotary part, and v): requested first, stored last, so
    // that the token's row is on its way while the sines and cosines are made
    const int k_tail = chunks - 2 * groups;             // chunks per k head that pass through
    const int n_copy = store ? a.n_kv_heads * (k_tail + chunks) : 0;
    auto copy_src = [&](int x) -> const bf16* {
        const int kvh = x / (k_tail + chunks), c = x % (k_tail + chunks);
        return c < k_tail ? row + a.k_off + kvh * hd + 2 * half + c * 8 : row + a.v_off + kvh * hd + (c - k_tail) * 8;
    };
    auto copy_dst = [&](int x) -> bf16* {
        const int kvh = x / (k_tail + chunks), c = x % (k_tail + chunks);
        return c < k_tail ? (bf16*)a.k_pool + cache_off + (size_t)kvh * a.page_rows * hd + 2 * half + c * 8
                          : (bf16*)a.v_pool + cache_off + (size_t)kvh * a.page_rows * hd + (c - k_tail) * 8;
    };
    constexpr int HELD = 4;                             // copied chunks a lane holds in registers (more go round a loop at the end)
    uint4 held[HELD];
#pragma unroll
    for (int i = 0; i < HELD; i++)
        if (lane + 32 * i < n_copy) held[i] = *(const uint4*)copy_src(lane + 32 * i);
    // ---- rotated part of q and k heads: work items (head slot, group of eight pairs)
    if (groups > 0) {
        const int lanes_per_head = groups < 32 ? groups : 32;          // groups <= 16 for head_dim <= 256
        const int heads_at_once = 32 / lanes_per_head;
        const int g = lane % lanes_per_head, h0 = lane / lanes_per_head;
        if (h0 < heads_at_once) {
            // four head slots at a time: their loads are requested together, and the next four before these are
            // worked on, so that a warp waits for memory once and not once per head
            auto fetch = [&](int hs0, uint4* wlo, uint4* whi) {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int hs = hs0 + u * heads_at_once;
                    if (hs < qk_slots) {
                        const int col0 = hs < a.n_heads ? a.q_off + hs * hd : a.k_off + (hs - a.n_heads) * hd;
                        wlo[u] = *(const uint4*)(row + col0 + g * 8);
                        whi[u] = *(const uint4*)(row + col0 + half + g * 8);
                    }
                }
            };
            uint4 wlo[4], whi[4], nlo[4], nhi[4];
            fetch(h0, wlo, whi);
            float sn[8], cs[8];
#pragma unroll
            for (int e = 0; e < 8; e++) sincosf((float)pos * a.inv_freq[g * 8 + e], &sn[e], &cs[e]);
            for (int hs0 = h0; hs0 < qk_slots; hs0 += 4 * heads_at_once) {
                fetch(hs0 + 4 * heads_at_once, nlo, nhi);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int hs = hs0 + u * heads_at_once;
                    if (hs < qk_slots) {
                        const bool is_q = hs < a.n_heads;
                        const int col0 = is_q ? a.q_off + hs * hd : a.k_off + (hs - a.n_heads) * hd;
                        float x0[8], x1[8], y0[8], y1[8];
                        unpack(wlo[u], x0); unpack(whi[u], x1);
#pragma unroll
                        for (int e = 0; e < 8; e++) { y0[e] = x0[e] * cs[e] - x1[e] * sn[e]; y1[e] = x1[e] * cs[e] + x0[e] * sn[e]; }
                        const uint4 w0 = pack(y0), w1 = pack(y1);
                        *(uint4*)(row + col0 + g * 8) = w0;
                        *(uint4*)(row + col0 + half + g * 8) = w1;
                        if (!is_q && store) {
                            bf16* dst = (bf16*)a.k_pool + cache_off + (size_t)(hs - a.n_heads) * a.page_rows * hd;
                            *(uint4*)(dst + g * 8) = w0;
                            *(uint4*)(dst + half + g * 8) = w1;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) { wlo[u] = nlo[u]; whi[u] = nhi[u]; }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < HELD; i++)
        if (lane + 32 * i < n_copy) *(uint4*)copy_dst(lane + 32 * i) = held[i];
    for (int x = lane + 32 * HELD; x < n_copy; x += 32) *(uint4*)copy_dst(x) = *(const uint4*)copy_src(x);
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
    // many tokens in bfloat16 with 16-byte aligned rows and heads: the warp-per-token kernel
    if (dtype == TB_BF16 && n_tokens >= 128 && a.partial == nullptr && a.head_dim % 16 == 0 &&
        (a.inv_freq == nullptr || a.rotary_dim == 0 || a.rotary_dim % 16 == 0) && a.rotary_dim / 16 <= 32 &&
        a.row_stride % 8 == 0 && a.q_off % 8 == 0 && a.k_off % 8 == 0 && a.v_off % 8 == 0 && ((uintptr_t)a.qkv & 15) == 0 &&
        ((uintptr_t)a.k_pool & 15) == 0 && ((uintptr_t)a.v_pool & 15) == 0) {
        RopeKvArgs b = a;
        if (b.inv_freq == nullptr) b.rotary_dim = 0;
        tb_launch(rope_kv_rows_kernel, dim3((n_tokens + 7) / 8), dim3(256), 0, stream, b, n_tokens);
        return tb_launch_status();
    }
    const int slots = a.n_heads + 2 * a.n_kv_heads;
    int tx = 16;                                     // threads over pairs (two pairs each)
    while (tx < 128 && tx * 4 < a.head_dim) tx <<= 1;
    int ty = 1;                                      // threads over head slots
    while (ty * 2 <= slots && tx * ty * 2 <= 256) ty <<= 1;
    // few tokens (decode): spread the head slots over several CTAs per token; many tokens: one CTA each,
    // so that the sines and cosines are computed once per token
    int gy = 1;
    if (n_tokens < 128) gy = (slots + ty - 1) / ty;
    if (gy > 65535) gy = 65535;
    TB_DISPATCH_1(dtype, T, tb_launch(rope_kv_kernel<T>, dim3(n_tokens, gy), dim3(tx, ty), 0, stream, a));
    return tb_launch_status();
}

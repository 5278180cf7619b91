/* The argument block of the decode attention entry points (tb_attn_decode, tb_attn_decode_lanes,
 * tb_attn_decode_stream, tb_attn_decode_noalloc, tb_attn_decode_simt).  Plain C, so that a C program can
 * fill it; the kernel files include this header, and the Python side mirrors it field by field
 * (a test compares the sizes).
 *
 * All pointers are device pointers.  "pools" are [pages][n_kv_heads][page_rows][hd] in the
 * activations' dtype; page_rows is 64.
 */
#ifndef TB_DECODE_ARGS_H
#define TB_DECODE_ARGS_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct DecodeArgs {
    const void* q;              /* [batch] rows of n_heads * hd, heads contiguous (ignored if qkv_part is set) */
    long long q_stride;         /* elements between two rows of q */
    const void* k_pool;         /* keys of one cache line */
    const void* v_pool;         /* values of one cache line */
    const int* page_table;      /* [batch][pt_stride]: page p of sequence b is pool page page_table[b][p] */
    int pt_stride;
    const int* len_after;       /* [batch] keys in the cache, the new token included */
    void* out;                  /* [batch, n_heads * hd] */
    float* partial;             /* scratch [batch, n_heads, n_splits, hd + 2] when n_splits > 1
                                   (tb_attn_decode_noalloc ignores it and uses its own) */
    int n_heads, n_kv_heads, hd, page_rows;
    int ring_rows;              /* 0: row = position; else the line is a ring, row = position mod ring_rows */
    int window;                 /* 0: every earlier key is visible; W: the last W keys, the query's own included */
    int n_splits;               /* pieces each sequence's keys are cut into */
    float scale;                /* scores are (q . k) * scale */
    float cap;                  /* 0: off; else scores become cap * tanh(score / cap) */
    int* tickets;               /* [batch, n_kv_heads] zeros, or null: with it the tensor-core kernel folds its
                                   splits itself (the last CTA to finish) and leaves the counters at zero */
    /* Tensor-core kernel only.  If qkv_part is set, q is not read: the step's q, k and v rows are taken from
     * these 32-bit partial sums of the q/k/v product ([qkv_splits][batch][row], columns: q heads, k heads,
     * v heads), added in split order; q and k are rotated (rotate-half pairing over the first rotary_dim dims;
     * none if inv_freq is null) at position len_after - 1 and rounded to bfloat16; k and v are also written to
     * their cache row. */
    const float* qkv_part;
    int qkv_splits;
    long long qkv_split_stride, qkv_row_stride;
    const float* inv_freq;      /* [rotary_dim / 2] */
    int rotary_dim;
} DecodeArgs;

#define TB_DECODE_ARGS_BYTES 168

#ifdef __cplusplus
}
static_assert(sizeof(DecodeArgs) == TB_DECODE_ARGS_BYTES, "DecodeArgs changed: update the Python mirror too");
#endif

#endif

/* Parts from outside the library, for the native host: a mixer or a feed-forward written in C, C++ or CUDA is
 * described by a table of functions and registered under a kind name; a model spec that names that kind is then built, bound
 * and stepped like any other, with no change to the library.  (The Python host takes parts written in Python
 * the same way, trapetum_b200.parts.register_part.)
 *
 * All pointers in tb_part_ctx are device pointers unless said otherwise; all work goes onto ctx->stream.
 * Every function returns 0 on success; on failure it may leave a message with ctx-free storage duration in
 * *error (a static string).
 */
#ifndef TRAPETUM_B200_PLUGIN_H
#define TRAPETUM_B200_PLUGIN_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { TB_DTYPE_F32 = 0, TB_DTYPE_BF16 = 1, TB_DTYPE_I32 = 2 };
enum { TB_NEED_NONE = 0, TB_NEED_KV = 1, TB_NEED_STATE = 2 };

typedef struct tb_tensor_decl {
    char name[192];             /* full tensor name (the part gets its prefix when it is made) */
    long long shape[4];
    int ndim;
    char role[16];              /* "matrix", "embedding", "norm" (random mode: the other std), "table" */
    int optional;
} tb_tensor_decl;

typedef struct tb_cache_need {
    int kind;                   /* TB_NEED_* */
    int n_kv_heads, head_dim, window;      /* TB_NEED_KV (window 0: every token is kept) */
    long long state_bytes;      /* TB_NEED_STATE: bytes per sequence, zeroed when a sequence starts */
} tb_cache_need;

/* What a mixer call may know about the running step. */
typedef struct tb_part_ctx {
    void* stream;               /* cudaStream_t */
    int dry;                    /* 1: the step is only being sized: call alloc as usual, launch and copy nothing */
    int is_prefill;             /* every sequence starts (whole prompts), else one token each */
    int n_tokens, batch;
    const int* positions;       /* [tokens] position of each token in its sequence */
    const int* token_seq;       /* [tokens] index of each token's sequence in the batch */
    const int* seq_start;       /* [batch + 1] first row of each sequence in the packed tokens */
    const int* len_after;       /* [batch] tokens of each sequence once this step is done */
    const int* slot_ids;        /* [batch] cache slot of each sequence */
    const int* host_slots;      /* the same on the host */
    const int* host_seq_lens;   /* [batch] tokens this step brings per sequence, on the host */
    void* state;                /* TB_NEED_STATE: [max_slots][state_bytes], a sequence's state at its slot */
    long long state_bytes;
    void* k;                    /* TB_NEED_KV: this call's cache line [pages][kv_heads][64][head_dim] */
    void* v;
    const int* page_table;      /* [batch][pt_stride]: page p of sequence b is pool page page_table[b][p] */
    int pt_stride, ring_rows;
    int line_owner;             /* this call writes the line (else it only reads another call's) */
    void* (*alloc)(void* arena, size_t bytes);      /* scratch that lives until the end of this layer */
    void* arena;
} tb_part_ctx;

typedef struct tb_mixer_plugin {
    /* params_json: the part spec's parameters; prefix: the layer's tensor-name prefix; dtype: the engine's compute dtype */
    void* (*create)(const char* params_json, const char* prefix, int dtype, const char** error);
    void (*destroy)(void* self);
    int (*tensor_count)(void* self);
    int (*tensor_decl)(void* self, int i, tb_tensor_decl* out);
    /* called once per declared tensor that was loaded; the memory stays the library's and outlives the part */
    int (*bind)(void* self, const char* name, const void* data, int dtype, const char** error);
    int (*cache_need)(void* self, tb_cache_need* out);
    /* x [rows, cols] in the compute dtype -> out [rows, cols] float32, the branch output */
    int (*forward)(void* self, const tb_part_ctx* ctx, const void* x, int x_dtype, long long rows, long long cols, float* out,
                   const char** error);
    int graph_safe;             /* 1: no launch depends on host values of the step (it may be captured into a graph) */
} tb_mixer_plugin;

/* Makes `kind` a mixer that model specs can name.  The table must outlive the process's models. */
int tb_register_mixer(const char* kind, const tb_mixer_plugin* plugin);

/* Makes `kind` a feed-forward.  The table is the same; cache_need is not asked (a feed-forward keeps nothing
 * between steps), and the cache fields of tb_part_ctx (state, k, v, page_table) are null in its calls. */
int tb_register_feed_forward(const char* kind, const tb_mixer_plugin* plugin);

#ifdef __cplusplus
}
#endif

#endif

/* trapetum_b200: the C interface of the native host.
 *
 * From a model folder (config.json + safetensors) to generated tokens on one GPU, in the manner of the
 * reference's C interface (runtime/include/trapetum.h:17-29: a session made from a folder, generate with a
 * per-token callback, free), with the step function, the cache's slots and random weights beside it.
 *
 *   tb_model* m = tb_model_load("folder", NULL, "bfloat16", 0);
 *   tb_engine* e = tb_engine_new(m, 8192, 0, 1);
 *   tb_generate(e, prompt, &len, 1, &params, NULL, -1, 64, on_token, user, out, out_len, 256);
 *
 * Every function that can fail returns a status (0 = done) or a null handle; tb_last_error() then tells why,
 * per thread.  Nothing throws across this interface.  Token ids are int32; logits are float32.
 */
#ifndef TRAPETUM_B200_H
#define TRAPETUM_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tb_model tb_model;
typedef struct tb_engine tb_engine;

enum { TB_OK = 0, TB_ERROR = 1, TB_STEP_ERROR = 2, TB_CACHE_FULL = 3, TB_STOPPED = 4 };

const char* tb_last_error(void);

/* Where the kernel libraries and their manifest.json lie (default: $TRAPETUM_KERNEL_DIR, else this library's folder). */
int tb_set_kernel_dir(const char* dir);

/* Decode attention's partition: 0 chosen per launch (the default), 1 every sequence cut into pieces, 2 all pages dealt
 * out as one stream.  For tests and comparisons; set it before an engine captures its decode graphs.  Returns the
 * previous setting. */
int tb_set_decode_partition(int mode);

/* A model from a folder.  spec_json: the model spec as the Python side serialises it, or NULL to build it here from
 * config.json (architectures this host knows by itself: Gemma2ForCausalLM).  dtype: "bfloat16" or "float32" (a true
 * 32-bit path).  fp16: what happens to float16 tensors in a bfloat16 engine: "widen" (NULL), "round" or "refuse". */
tb_model* tb_model_load(const char* folder, const char* spec_json, const char* dtype, int device, const char* fp16);
/* A model with random weights made on the device: the values that the random-weights mode stores for this seed.
 * config_or_spec_json: a config.json's text, or a spec. */
tb_model* tb_model_random(const char* config_or_spec_json, unsigned long long seed, float std, float norm_std,
                          const char* dtype, int device);
void tb_model_free(tb_model* m);
int tb_model_vocab(const tb_model* m);
int tb_model_max_positions(const tb_model* m);
/* 1 if every part kind of the spec has a native class (0: tb_last_error names the first that has not). */
int tb_spec_is_native(const char* spec_json);

/* max_tokens: the most tokens that live sequences hold at any time, each rounded up to 64.  max_slots 0: default. */
tb_engine* tb_engine_new(tb_model* m, long long max_tokens, int max_slots, int use_graphs);
void tb_engine_free(tb_engine* e);
/* Run on the caller's stream (a cudaStream_t; 0 is the legacy default stream) instead of the engine's own. */
int tb_engine_set_stream(tb_engine* e, void* stream);
int tb_engine_synchronize(tb_engine* e);

/* Slots for n sequences that start together; tb_release gives slots and pages back. */
int tb_start(tb_engine* e, int n, int* slots_out);
int tb_release(tb_engine* e, const int* slots, int n);

/* One step.  tokens: the sequences' new tokens back to back, n_new[i] of sequence i (whole prompts for sequences
 * that all start, or one token each).  want / n_want: per sequence, the places among its tokens of this step whose
 * logits are returned, in order (want NULL: each sequence's last token).  greedy 0: *out_logits is set to a device
 * pointer to float32 [*out_rows, vocab]; greedy 1: *out_ids to int32 [*out_rows], the largest logit's id (the
 * smallest id on a tie).  Both stay valid until the engine's next call; the work is queued on the engine's stream. */
int tb_step(tb_engine* e, const int* slots, int n_seqs, const int* tokens, const int* n_new, const int* want,
            const int* n_want, int greedy, const float** out_logits, const int** out_ids, int* out_rows);
/* The same, with the logits copied to host memory of the caller's (rows * vocab floats; capacity in floats). */
int tb_step_host(tb_engine* e, const int* slots, int n_seqs, const int* tokens, const int* n_new, const int* want,
                 const int* n_want, float* out_logits, long long capacity, int* out_rows);

/* One step of a generation loop: the tokens in, each sequence's greedy next token out (host memory, one id per
 * sequence: the largest logit at its last token of this step).  Returns when the ids have arrived. */
int tb_step_tokens(tb_engine* e, const int* slots, int n_seqs, const int* tokens, const int* n_new, int* out_ids);

typedef struct tb_sampling {
    float temperature;              /* <= 0: greedy */
    float top_p;                    /* default 0.95 */
    float repetition_penalty;       /* default 1.0 (> 1 penalises the last 128 tokens) */
    int max_tokens;                 /* new tokens per request */
    unsigned long long seed;
} tb_sampling;

/* Called for every emitted token; a non-zero return ends the generation (tb_generate then returns TB_STOPPED). */
typedef int (*tb_on_token)(int request, int token, void* user);

/* Generate for n_prompts prompts (back to back in `prompts`, prompt_lens[i] tokens each), in as many batches as
 * the cache needs.  stop_ids: n_stop ids that end a sequence and are not emitted (n_stop -1: the model's own).
 * out_tokens: n_prompts rows of out_capacity ids; out_lens[i] new tokens were written to row i. */
int tb_generate(tb_engine* e, const int* prompts, const int* prompt_lens, int n_prompts, const tb_sampling* params,
                const int* stop_ids, int n_stop, int max_batch, tb_on_token on_token, void* user, int* out_tokens,
                int* out_lens, int out_capacity);

/* Looking into the cache (tests, tools). */
int tb_cache_groups(tb_engine* e);
int tb_cache_group_info(tb_engine* e, int group, void** k, void** v, int* lines, int* pages, int* kv_heads,
                        int* head_dim, int* ring_rows, int* dtype_code);
int tb_cache_max_slots(tb_engine* e);
long long tb_cache_max_tokens(tb_engine* e);
long long tb_cache_length(tb_engine* e, int slot);                      /* -1: not held */
int tb_cache_pages(tb_engine* e, int slot, int group, int* out, int capacity);   /* returns the count, -1 on error */
int tb_cache_live(tb_engine* e, int* out, int capacity);                /* returns the count */
int tb_cache_check(tb_engine* e);
int tb_cache_grow(tb_engine* e, const int* slots, const int* growth, int n);     /* room without a step (measurements) */

/* What needs no GPU (tools, tests).
 * tb_spec_from_config: the spec this host builds from a config.json's text (NULL on error).
 * tb_check_weights: holds a folder's weight files against a spec; TB_OK, or TB_ERROR with one message that lists
 * everything that does not fit.
 * tb_plan_batches: cuts requests into batches as tb_generate does; batch_of[i] is request i's batch; returns the
 * number of batches, -1 on error.
 * tb_decode_launch_shape: what a decode step's launches depend on, for a batch with these lengths after the step:
 * out3 = {length bucket, unevenness of the lengths (0..3), pieces a sequence's pages are cut into}; returns 1 if the
 * pages are dealt out as one stream instead, 0 if not, -1 on error.
 * tb_sim_cache_*: the cache's bookkeeping without storage.  needs_json: [{"entry", "n_kv_heads", "head_dim",
 * "window" (0: none)} or {"entry", "state_bytes"}, ...]. */
const char* tb_spec_from_config(const char* config_json);
int tb_check_weights(const char* folder, const char* spec_json, const char* dtype, const char* fp16);
int tb_plan_batches(const int* prompt_lens, int n, int max_new, int max_batch, long long max_tokens, int max_positions,
                    int* batch_of);
int tb_decode_launch_shape(const int* lens_after, int n, int n_kv_heads, int ring_rows, int sms, int* out3);
typedef struct tb_sim_cache tb_sim_cache;
tb_sim_cache* tb_sim_cache_new(const char* needs_json, long long max_tokens, int max_slots);
void tb_sim_cache_free(tb_sim_cache* c);
int tb_sim_cache_claim(tb_sim_cache* c);                                         /* the slot, -1 on error */
int tb_sim_cache_grow(tb_sim_cache* c, const int* slots, const int* growth, int n);
int tb_sim_cache_shrink(tb_sim_cache* c, const int* slots, const int* growth, int n);
int tb_sim_cache_release(tb_sim_cache* c, int slot);
int tb_sim_cache_check(tb_sim_cache* c);
long long tb_sim_cache_length(tb_sim_cache* c, int slot);
int tb_sim_cache_pages(tb_sim_cache* c, int slot, int group, int* out, int capacity);
int tb_sim_cache_groups(tb_sim_cache* c);
long long tb_sim_cache_epoch(tb_sim_cache* c);

/* "" when no kernel's bounded wait has run out since the last call; synchronises. */
const char* tb_kernel_errors(tb_engine* e);
long long tb_kernel_launches(void);
int tb_graphs_captured(tb_engine* e);
long long tb_last_h2d_bytes(tb_engine* e);

#ifdef __cplusplus
}
#endif

#endif

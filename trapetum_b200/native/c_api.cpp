// The C interface of the native host (see trapetum_b200.h): every function catches what the C++ below it throws
// and turns it into a status and a message.
#include "trapetum_b200.h"
#include "plugin.h"

#include "engine.hpp"

using namespace tb;

struct tb_model {
    std::unique_ptr<Model> m;
};
struct tb_engine {
    std::unique_ptr<Engine> e;
    std::string errors;
};

static thread_local std::string g_error;

static int fail(const std::exception& ex) {
    g_error = ex.what();
    if (dynamic_cast<const StepError*>(&ex)) return TB_STEP_ERROR;
    if (dynamic_cast<const CacheFull*>(&ex)) return TB_CACHE_FULL;
    return TB_ERROR;
}
#define TB_TRY try {
#define TB_CATCH_STATUS } catch (const std::exception& ex) { return fail(ex); } catch (...) { g_error = "unknown error"; return TB_ERROR; }
#define TB_CATCH_NULL } catch (const std::exception& ex) { fail(ex); return nullptr; } catch (...) { g_error = "unknown error"; return nullptr; }

static DType parse_dtype(const char* d) {
    const std::string s = d ? d : "bfloat16";
    if (s == "bfloat16" || s == "bf16") return BF16;
    if (s == "float32" || s == "fp32") return F32;
    throw Error("unknown dtype '" + s + "' (bfloat16 or float32)");
}

// An Ops for work outside any engine (binding and making weights): the default stream, no arena.
static Ops loader_ops() {
    Ops o;
    static Arena none;
    o.arena = &none;
    o.stream = nullptr;
    return o;
}

extern "C" {

const char* tb_last_error(void) { return g_error.c_str(); }

int tb_set_kernel_dir(const char* dir) {
    TB_TRY
    Kernels::get().set_dir(dir ? dir : "");
    return TB_OK;
    TB_CATCH_STATUS
}

tb_model* tb_model_load(const char* folder, const char* spec_json, const char* dtype, int device, const char* fp16) {
    TB_TRY
    if (!folder) throw Error("tb_model_load: no folder");
    cuda_ok(cudaSetDevice(device), "selecting the device");
    Json spec;
    if (spec_json && *spec_json) spec = Json::parse(spec_json);
    else {
        const std::string p = std::string(folder) + "/config.json";
        if (!file_exists(p)) throw Error("no config.json at " + p);
        Json cfg;
        try { cfg = Json::parse(read_text(p)); } catch (const Error& e) { throw Error(p + " is not valid JSON: " + e.what()); }
        spec = spec_for_config(cfg);
        add_generation_stop_ids(folder, spec);
    }
    std::unique_ptr<tb_model> h(new tb_model);
    h->m.reset(new Model(spec, parse_dtype(dtype), device));
    Ops ops = loader_ops();
    h->m->bind(load_tensors(folder, h->m->wanted(), h->m->rt.dt, fp16 && *fp16 ? fp16 : "widen"), ops);
    return h.release();
    TB_CATCH_NULL
}

tb_model* tb_model_random(const char* json, unsigned long long seed, float std_, float norm_std, const char* dtype, int device) {
    TB_TRY
    if (!json) throw Error("tb_model_random: no configuration");
    cuda_ok(cudaSetDevice(device), "selecting the device");
    Json j = Json::parse(json);
    Json spec = j.has("layers") && j.has("schedule") ? j : spec_for_config(j);
    std::unique_ptr<tb_model> h(new tb_model);
    h->m.reset(new Model(spec, parse_dtype(dtype), device));
    Ops ops = loader_ops();
    h->m->bind(random_tensors(h->m->wanted(), seed, std_, norm_std, h->m->rt.dt, ops), ops);
    return h.release();
    TB_CATCH_NULL
}

void tb_model_free(tb_model* m) { delete m; }
int tb_model_vocab(const tb_model* m) { return m ? m->m->vocab : 0; }
int tb_model_max_positions(const tb_model* m) { return m ? m->m->max_positions : 0; }

int tb_spec_is_native(const char* spec_json) {
    try {
        std::string why;
        if (Model::spec_is_native(Json::parse(spec_json ? spec_json : ""), &why)) return 1;
        g_error = "no native " + why;
    } catch (const std::exception& ex) {
        g_error = ex.what();
    }
    return 0;
}

tb_engine* tb_engine_new(tb_model* m, long long max_tokens, int max_slots, int use_graphs) {
    TB_TRY
    if (!m) throw Error("tb_engine_new: no model");
    std::unique_ptr<tb_engine> h(new tb_engine);
    h->e.reset(new Engine(*m->m, max_tokens, max_slots, use_graphs != 0));
    return h.release();
    TB_CATCH_NULL
}
void tb_engine_free(tb_engine* e) { delete e; }

int tb_engine_set_stream(tb_engine* e, void* stream) {
    TB_TRY
    e->e->set_stream((cudaStream_t)stream);
    return TB_OK;
    TB_CATCH_STATUS
}
int tb_engine_synchronize(tb_engine* e) {
    TB_TRY
    e->e->synchronize();
    return TB_OK;
    TB_CATCH_STATUS
}

int tb_start(tb_engine* e, int n, int* slots_out) {
    TB_TRY
    auto s = e->e->start(n);
    std::copy(s.begin(), s.end(), slots_out);
    return TB_OK;
    TB_CATCH_STATUS
}
int tb_release(tb_engine* e, const int* slots, int n) {
    TB_TRY
    e->e->release(std::vector<int>(slots, slots + n));
    return TB_OK;
    TB_CATCH_STATUS
}

static StepResult do_step(tb_engine* e, const int* slots, int n_seqs, const int* tokens, const int* n_new, const int* want,
                          const int* n_want, bool greedy) {
    if (n_seqs < 0) throw StepError("a step needs at least one sequence");
    std::vector<int> sl(slots, slots + n_seqs);
    std::vector<std::vector<int>> toks(n_seqs), wants(n_seqs);
    size_t t = 0, w = 0;
    for (int i = 0; i < n_seqs; i++) {
        if (n_new[i] < 0) throw StepError("a negative token count");
        toks[i].assign(tokens + t, tokens + t + n_new[i]);
        t += n_new[i];
        if (n_want) {
            if (n_want[i] < 0) throw StepError("a negative 'want' count");
            if (n_want[i]) wants[i].assign(want + w, want + w + n_want[i]);
            w += n_want[i];
        }
    }
    return e->e->step(sl, toks, n_want ? &wants : nullptr, greedy);
}

int tb_step(tb_engine* e, const int* slots, int n_seqs, const int* tokens, const int* n_new, const int* want, const int* n_want,
            int greedy, const float** out_logits, const int** out_ids, int* out_rows) {
    TB_TRY
    StepResult r = do_step(e, slots, n_seqs, tokens, n_new, want, n_want, greedy != 0);
    if (out_logits) *out_logits = r.logits;
    if (out_ids) *out_ids = r.ids;
    if (out_rows) *out_rows = r.rows;
    return TB_OK;
    TB_CATCH_STATUS
}

int tb_step_host(tb_engine* e, const int* slots, int n_seqs, const int* tokens, const int* n_new, const int* want,
                 const int* n_want, float* out_logits, long long capacity, int* out_rows) {
    TB_TRY
    StepResult r = do_step(e, slots, n_seqs, tokens, n_new, want, n_want, false);
    if (out_rows) *out_rows = r.rows;
    const long long n = (long long)r.rows * e->e->model.vocab;
    if (n > capacity) throw Error(fmt("tb_step_host: %lld floats of logits, room for %lld", n, capacity));
    if (n) cuda_ok(cudaMemcpyAsync(out_logits, r.logits, (size_t)n * 4, cudaMemcpyDeviceToHost, e->e->ops.stream), "reading the logits");
    e->e->synchronize();
    return TB_OK;
    TB_CATCH_STATUS
}

int tb_step_tokens(tb_engine* e, const int* slots, int n_seqs, const int* tokens, const int* n_new, int* out_ids) {
    TB_TRY
    StepResult r = do_step(e, slots, n_seqs, tokens, n_new, nullptr, nullptr, true);
    e->e->read_ids(r.ids, r.rows, out_ids);
    return TB_OK;
    TB_CATCH_STATUS
}

int tb_generate(tb_engine* e, const int* prompts, const int* prompt_lens, int n_prompts, const tb_sampling* params,
                const int* stop_ids, int n_stop, int max_batch, tb_on_token on_token, void* user, int* out_tokens,
                int* out_lens, int out_capacity) {
    TB_TRY
    std::vector<std::vector<int>> ps(n_prompts);
    size_t t = 0;
    for (int i = 0; i < n_prompts; i++) { ps[i].assign(prompts + t, prompts + t + prompt_lens[i]); t += prompt_lens[i]; }
    SamplingParams p;
    if (params) {
        p.temperature = params->temperature; p.top_p = params->top_p; p.repetition_penalty = params->repetition_penalty;
        p.max_tokens = params->max_tokens; p.seed = params->seed;
    }
    std::vector<int> stops;
    if (n_stop >= 0) stops.assign(stop_ids, stop_ids + n_stop);
    struct Watch { tb_on_token cb; void* user; bool stopped; } watch{on_token, user, false};
    auto outs = generate(*e->e, ps, p, n_stop >= 0 ? &stops : nullptr, max_batch > 0 ? max_batch : 64,
                         on_token ? [](int r, int tok, void* w) -> int {
                             Watch* x = (Watch*)w;
                             const int stop = x->cb(r, tok, x->user);
                             if (stop) x->stopped = true;
                             return stop;
                         } : (OnToken) nullptr, &watch);
    for (int i = 0; i < n_prompts; i++) {
        const int n = std::min<int>((int)outs[i].size(), out_capacity);
        if (out_tokens) std::copy(outs[i].begin(), outs[i].begin() + n, out_tokens + (size_t)i * out_capacity);
        if (out_lens) out_lens[i] = n;
    }
    return watch.stopped ? TB_STOPPED : TB_OK;
    TB_CATCH_STATUS
}

int tb_cache_groups(tb_engine* e) { return (int)e->e->cache->groups().size(); }
int tb_cache_group_info(tb_engine* e, int group, void** k, void** v, int* lines, int* pages, int* kv_heads, int* head_dim,
                        int* ring_rows, int* dtype_code) {
    TB_TRY
    auto& gs = e->e->cache->groups();
    if (group < 0 || group >= (int)gs.size()) throw Error("no such cache group");
    KVGroup& g = gs[group];
    if (k) *k = g.k.p;
    if (v) *v = g.v.p;
    if (lines) *lines = (int)g.entries.size();
    if (pages) *pages = g.n_pages;
    if (kv_heads) *kv_heads = g.n_kv_heads;
    if (head_dim) *head_dim = g.head_dim;
    if (ring_rows) *ring_rows = g.ring_rows;
    if (dtype_code) *dtype_code = (int)e->e->model.rt.dt;
    return TB_OK;
    TB_CATCH_STATUS
}
int tb_cache_max_slots(tb_engine* e) { return e->e->cache->max_slots(); }
long long tb_cache_max_tokens(tb_engine* e) { return e->e->cache->max_tokens(); }
long long tb_cache_length(tb_engine* e, int slot) { return e->e->cache->slot_held(slot) ? e->e->cache->length(slot) : -1; }
int tb_cache_pages(tb_engine* e, int slot, int group, int* out, int capacity) {
    try {
        const auto& pg = e->e->cache->pages(slot, group);
        for (size_t i = 0; i < pg.size() && (int)i < capacity; i++) out[i] = pg[i];
        return (int)pg.size();
    } catch (const std::exception& ex) {
        fail(ex);
        return -1;
    }
}
int tb_cache_live(tb_engine* e, int* out, int capacity) {
    auto v = e->e->cache->live_slots();
    for (size_t i = 0; i < v.size() && (int)i < capacity; i++) out[i] = v[i];
    return (int)v.size();
}
int tb_cache_check(tb_engine* e) {
    TB_TRY
    e->e->cache->check();
    return TB_OK;
    TB_CATCH_STATUS
}
int tb_cache_grow(tb_engine* e, const int* slots, const int* growth, int n) {
    TB_TRY
    e->e->cache->grow(std::vector<int>(slots, slots + n), std::vector<int>(growth, growth + n));
    return TB_OK;
    TB_CATCH_STATUS
}

int tb_register_mixer(const char* kind, const tb_mixer_plugin* plugin) {
    TB_TRY
    if (!kind || !*kind || !plugin || !plugin->create || !plugin->forward) throw Error("tb_register_mixer: a kind, create and forward are needed");
    register_builtin_parts();
    Registry<MixerPart>::add(kind, [plugin](const PartSpec& s, const std::string& prefix, Runtime rt) {
        return std::unique_ptr<MixerPart>(new PluginMixer(plugin, s, prefix, rt));
    });
    return TB_OK;
    TB_CATCH_STATUS
}

int tb_set_decode_partition(int mode) {
    const int was = Ops::decode_partition_override();
    Ops::decode_partition_override() = (mode == 1 || mode == 2) ? mode : 0;
    return was;
}

int tb_register_feed_forward(const char* kind, const tb_mixer_plugin* plugin) {
    TB_TRY
    if (!kind || !*kind || !plugin || !plugin->create || !plugin->forward)
        throw Error("tb_register_feed_forward: a kind, create and forward are needed");
    register_builtin_parts();
    Registry<FeedForwardPart>::add(kind, [plugin](const PartSpec& s, const std::string& prefix, Runtime rt) {
        return std::unique_ptr<FeedForwardPart>(new PluginFeedForward(plugin, s, prefix, rt));
    });
    return TB_OK;
    TB_CATCH_STATUS
}

const char* tb_spec_from_config(const char* config_json) {
    static thread_local std::string out;
    try {
        out = spec_for_config(Json::parse(config_json ? config_json : "")).dump();
        return out.c_str();
    } catch (const std::exception& ex) {
        fail(ex);
        return nullptr;
    }
}

int tb_check_weights(const char* folder, const char* spec_json, const char* dtype, const char* fp16) {
    TB_TRY
    Model m(Json::parse(spec_json ? spec_json : ""), parse_dtype(dtype), 0);
    check_tensors(folder ? folder : "", m.wanted(), m.rt.dt, fp16 && *fp16 ? fp16 : "widen");
    return TB_OK;
    TB_CATCH_STATUS
}

int tb_plan_batches(const int* prompt_lens, int n, int max_new, int max_batch, long long max_tokens, int max_positions, int* batch_of) {
    try {
        auto batches = plan_batches(std::vector<int>(prompt_lens, prompt_lens + n), max_new, max_batch, max_tokens, max_positions);
        for (size_t b = 0; b < batches.size(); b++)
            for (int i : batches[b]) batch_of[i] = (int)b;
        return (int)batches.size();
    } catch (const std::exception& ex) {
        fail(ex);
        return -1;
    }
}

int tb_decode_launch_shape(const int* lens_after, int n, int n_kv_heads, int ring_rows, int sms, int* out3) {
    try {
        if (n <= 0 || n_kv_heads <= 0 || sms <= 0) throw Error("tb_decode_launch_shape: a batch, kv heads and SMs are needed");
        std::vector<int> lens(lens_after, lens_after + n);
        const int bucket = len_bucket(*std::max_element(lens.begin(), lens.end()));
        const int rows = ring_rows ? std::min(bucket, ring_rows) : bucket;
        const int pages = std::max(1, (rows + PAGE_ROWS - 1) / PAGE_ROWS);
        const int uneven = unevenness(lens);
        const int splits = Ops::choose_decode_splits(n, n_kv_heads, pages, sms);
        out3[0] = bucket; out3[1] = uneven; out3[2] = splits;
        return Ops::decode_partition_is_stream(n, n_kv_heads, pages, splits, uneven, sms) ? 1 : 0;
    } catch (const std::exception& ex) {
        fail(ex);
        return -1;
    }
}

struct tb_sim_cache {
    std::unique_ptr<Cache> c;
};

tb_sim_cache* tb_sim_cache_new(const char* needs_json, long long max_tokens, int max_slots) {
    TB_TRY
    Json j = Json::parse(needs_json ? needs_json : "[]");
    std::map<int, CacheNeed> needs;
    for (auto& e : j.arr) {
        CacheNeed n;
        if (e.has("state_bytes")) { n.kind = CacheNeed::STATE; n.state_bytes = (size_t)e.at("state_bytes").integer("state_bytes"); }
        else {
            n.kind = CacheNeed::KV;
            n.n_kv_heads = (int)e.at("n_kv_heads").integer("n_kv_heads");
            n.head_dim = (int)e.at("head_dim").integer("head_dim");
            n.window = e.has("window") && !e.at("window").is_null() ? (int)e.at("window").integer("window") : 0;
        }
        needs[(int)e.at("entry").integer("entry")] = n;
    }
    std::unique_ptr<tb_sim_cache> h(new tb_sim_cache);
    h->c.reset(new Cache(needs, {}, max_tokens, BF16, max_slots, false));
    return h.release();
    TB_CATCH_NULL
}
void tb_sim_cache_free(tb_sim_cache* c) { delete c; }
int tb_sim_cache_claim(tb_sim_cache* c) {
    try { return c->c->claim(); } catch (const std::exception& ex) { fail(ex); return -1; }
}
int tb_sim_cache_grow(tb_sim_cache* c, const int* slots, const int* growth, int n) {
    TB_TRY
    c->c->grow(std::vector<int>(slots, slots + n), std::vector<int>(growth, growth + n));
    return TB_OK;
    TB_CATCH_STATUS
}
int tb_sim_cache_shrink(tb_sim_cache* c, const int* slots, const int* growth, int n) {
    TB_TRY
    c->c->shrink(std::vector<int>(slots, slots + n), std::vector<int>(growth, growth + n));
    return TB_OK;
    TB_CATCH_STATUS
}
int tb_sim_cache_release(tb_sim_cache* c, int slot) {
    TB_TRY
    c->c->release(slot);
    return TB_OK;
    TB_CATCH_STATUS
}
int tb_sim_cache_check(tb_sim_cache* c) {
    TB_TRY
    c->c->check();
    return TB_OK;
    TB_CATCH_STATUS
}
long long tb_sim_cache_length(tb_sim_cache* c, int slot) { return c->c->slot_held(slot) ? c->c->length(slot) : -1; }
int tb_sim_cache_pages(tb_sim_cache* c, int slot, int group, int* out, int capacity) {
    try {
        const auto& pg = c->c->pages(slot, group);
        for (size_t i = 0; i < pg.size() && (int)i < capacity; i++) out[i] = pg[i];
        return (int)pg.size();
    } catch (const std::exception& ex) { fail(ex); return -1; }
}
int tb_sim_cache_groups(tb_sim_cache* c) { return (int)c->c->groups().size(); }
long long tb_sim_cache_epoch(tb_sim_cache* c) { return c->c->epoch; }

const char* tb_kernel_errors(tb_engine* e) {
    try {
        e->errors = e->e->kernel_errors();
    } catch (const std::exception& ex) {
        e->errors = ex.what();
    }
    return e->errors.c_str();
}
long long tb_kernel_launches(void) { return Kernels::get().launches; }
int tb_graphs_captured(tb_engine* e) { return e->e->graphs_captured(); }
long long tb_last_h2d_bytes(tb_engine* e) { return e->e->h2d_bytes_last; }

}  // extern "C"

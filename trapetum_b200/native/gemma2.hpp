// Gemma-2 as data, natively: its config.json turned into the model spec that the parts are built from.  Nothing
// here computes.  Keys and defaults follow what the reference's exporter reads from the model's config object
// (model/export_gemma.py:40-46); the reference asserts query_pre_attn_scalar == head_dim and widths that are
// multiples of 256 (:47-49); neither restriction exists here.  The Python side makes the same spec
// (trapetum_b200/models/gemma2.py); this copy lets a C program load a Gemma-2 folder with no Python around.
#pragma once
#include "model.hpp"

namespace tb {

namespace cfgkey {
inline long long integer(const Json& d, const std::string& k, long long def, bool has_def) {
    const Json* v = d.find(k);
    if (!v || v->is_null()) {
        if (has_def) return def;
        throw Error("config.json: key '" + k + "' is missing");
    }
    if (v->kind != Json::Num || !v->is_int) throw Error("config.json: key '" + k + "' must be an integer");
    return v->i;
}
inline double number(const Json& d, const std::string& k, double def, bool has_def, bool* absent = nullptr) {
    const Json* v = d.find(k);
    if (absent) *absent = !v || v->is_null();
    if (!v || v->is_null()) {
        if (has_def) return def;
        throw Error("config.json: key '" + k + "' is missing");
    }
    if (v->kind != Json::Num) throw Error("config.json: key '" + k + "' must be a number");
    return v->num;
}
inline std::vector<int> id_list(const Json& d, const std::string& k) {
    std::vector<int> out;
    const Json* v = d.find(k);
    if (!v || v->is_null()) return out;
    if (v->kind == Json::Num && v->is_int) out.push_back((int)v->i);
    else if (v->kind == Json::Arr) {
        for (auto& x : v->arr) {
            if (x.kind != Json::Num || !x.is_int) throw Error("config.json: key '" + k + "' must be an integer or a list of integers");
            out.push_back((int)x.i);
        }
    } else throw Error("config.json: key '" + k + "' must be an integer or a list of integers");
    return out;
}
}  // namespace cfgkey

inline Json part(const std::string& kind, Json params) {
    Json p = Json::make_obj();
    p.set("kind", Json::make_str(kind));
    p.set("params", std::move(params));
    return p;
}

inline Json gemma2_spec(const Json& d) {
    using namespace cfgkey;
    const long long L = integer(d, "num_hidden_layers", 0, false), H = integer(d, "hidden_size", 0, false);
    const long long nh = integer(d, "num_attention_heads", 0, false), nkv = integer(d, "num_key_value_heads", nh, true);
    const long long hd = integer(d, "head_dim", 0, false), I = integer(d, "intermediate_size", 0, false);
    const long long V = integer(d, "vocab_size", 0, false), max_pos = integer(d, "max_position_embeddings", 8192, true);
    const double eps = number(d, "rms_norm_eps", 1e-6, true), theta = number(d, "rope_theta", 10000.0, true);
    bool no_window = false, no_acap = false, no_fcap = false;
    const long long window = (long long)number(d, "sliding_window", 0, true, &no_window);
    const double qpas = number(d, "query_pre_attn_scalar", (double)hd, true);
    double attn_cap = number(d, "attn_logit_softcapping", 0, true, &no_acap);
    double final_cap = number(d, "final_logit_softcapping", 0, true, &no_fcap);
    std::string act = "gelu_pytorch_tanh";
    for (const char* k : {"hidden_act", "hidden_activation"})
        if (const Json* v = d.find(k))
            if (v->kind == Json::Str) act = v->str;
    const Json* tie_j = d.find("tie_word_embeddings");
    const bool tie = !tie_j || tie_j->is_null() || tie_j->truthy();
    const std::pair<const char*, long long> positive[] = {{"num_hidden_layers", L}, {"hidden_size", H}, {"num_attention_heads", nh},
        {"num_key_value_heads", nkv}, {"head_dim", hd}, {"intermediate_size", I}, {"vocab_size", V}, {"max_position_embeddings", max_pos}};
    for (auto& kv : positive)
        if (kv.second <= 0) throw Error(fmt("config.json: key '%s' must be positive, got %lld", kv.first, kv.second));
    if (nh % nkv) throw Error(fmt("config.json: 'num_attention_heads' (%lld) must be a multiple of 'num_key_value_heads' (%lld)", nh, nkv));
    if (hd % 2) throw Error(fmt("config.json: 'head_dim' (%lld) must be even (rotary pairs)", hd));
    if (!(eps > 0)) throw Error("config.json: 'rms_norm_eps' must be positive");
    if (!(theta > 0)) throw Error("config.json: 'rope_theta' must be positive");
    if (!(qpas > 0)) throw Error("config.json: 'query_pre_attn_scalar' must be positive");
    if (!no_window && window <= 0) throw Error("config.json: 'sliding_window' must be positive or null");
    if (attn_cap < 0) attn_cap = 0;          // 0 means "off", as in the exporter's `or 0.0` (model/export_gemma.py:44-45)
    if (final_cap < 0) final_cap = 0;
    if (act != "gelu_pytorch_tanh") throw Error("config.json: 'hidden_activation' is '" + act + "'; this architecture computes gelu_pytorch_tanh only");
    std::vector<bool> sliding((size_t)L);
    const Json* lt = d.find("layer_types");
    for (long long i = 0; i < L; i++) {
        if (lt && !lt->is_null()) {
            if (lt->kind != Json::Arr || (long long)lt->arr.size() != L) throw Error(fmt("config.json: 'layer_types' must list %lld entries", L));
            const std::string& t = lt->arr[(size_t)i].string("layer_types entry");
            if (t != "sliding_attention" && t != "full_attention") throw Error("config.json: 'layer_types' entries are sliding_attention or full_attention");
            sliding[(size_t)i] = t == "sliding_attention";
        } else sliding[(size_t)i] = (i % 2 == 0);          // Gemma-2's rule: layers with an even index slide
        if (no_window) sliding[(size_t)i] = false;
    }
    auto norm = [&](const std::string& name) {
        Json p = Json::make_obj();
        p.set("size", Json::make_int(H)); p.set("eps", Json::make_num(eps)); p.set("unit_offset", Json::make_bool(true));
        p.set("weight", Json::make_str(name));
        return part("rmsnorm", p);
    };
    Json spec = Json::make_obj();
    spec.set("architecture", Json::make_str("Gemma2ForCausalLM"));
    spec.set("hidden_size", Json::make_int(H));
    spec.set("vocab_size", Json::make_int(V));
    Json emb = Json::make_obj();
    emb.set("vocab_size", Json::make_int(V)); emb.set("hidden_size", Json::make_int(H));
    emb.set("scale", Json::make_num(std::sqrt((double)H))); emb.set("weight", Json::make_str("model.embed_tokens.weight"));
    spec.set("embedding", part("embedding", emb));
    Json layers = Json::make_arr(), sched = Json::make_arr();
    for (long long i = 0; i < L; i++) {
        Json pos = Json::make_obj();
        pos.set("head_dim", Json::make_int(hd)); pos.set("theta", Json::make_num(theta)); pos.set("rotary_dim", Json::make_int(hd));
        Json mx = Json::make_obj();
        mx.set("hidden_size", Json::make_int(H)); mx.set("num_heads", Json::make_int(nh)); mx.set("num_kv_heads", Json::make_int(nkv));
        mx.set("head_dim", Json::make_int(hd)); mx.set("scale", Json::make_num(std::pow(qpas, -0.5)));
        mx.set("softcap", attn_cap > 0 ? Json::make_num(attn_cap) : Json());
        mx.set("window", sliding[(size_t)i] ? Json::make_int(window) : Json());
        mx.set("position", part("rope", pos));
        mx.set("q", Json::make_str("self_attn.q_proj.weight")); mx.set("k", Json::make_str("self_attn.k_proj.weight"));
        mx.set("v", Json::make_str("self_attn.v_proj.weight")); mx.set("o", Json::make_str("self_attn.o_proj.weight"));
        Json ff = Json::make_obj();
        ff.set("hidden_size", Json::make_int(H)); ff.set("intermediate_size", Json::make_int(I)); ff.set("activation", Json::make_str("gelu_tanh"));
        ff.set("gate", Json::make_str("mlp.gate_proj.weight")); ff.set("up", Json::make_str("mlp.up_proj.weight"));
        ff.set("down", Json::make_str("mlp.down_proj.weight"));
        Json bl = Json::make_obj();
        bl.set("pre_mixer_norm", norm("input_layernorm.weight")); bl.set("post_mixer_norm", norm("post_attention_layernorm.weight"));
        bl.set("pre_ffn_norm", norm("pre_feedforward_layernorm.weight")); bl.set("post_ffn_norm", norm("post_feedforward_layernorm.weight"));
        Json layer = Json::make_obj();
        layer.set("prefix", Json::make_str(fmt("model.layers.%lld.", i)));
        layer.set("block", part("sandwich", bl)); layer.set("mixer", part("attention", mx)); layer.set("feed_forward", part("gated_mlp", ff));
        layers.arr.push_back(std::move(layer));
        Json e = Json::make_obj();
        e.set("layer", Json::make_int(i)); e.set("cache_of", Json());
        sched.arr.push_back(std::move(e));
    }
    spec.set("layers", std::move(layers));
    spec.set("schedule", std::move(sched));
    spec.set("final_norm", norm("model.norm.weight"));
    Json head = Json::make_obj();
    head.set("vocab_size", Json::make_int(V)); head.set("hidden_size", Json::make_int(H));
    head.set("softcap", final_cap > 0 ? Json::make_num(final_cap) : Json());
    head.set("weight", Json::make_str("lm_head.weight"));
    head.set("tied_to", tie ? Json::make_str("model.embed_tokens.weight") : Json());
    spec.set("head", part("linear_head", head));
    spec.set("max_positions", Json::make_int(max_pos));
    Json stops = Json::make_arr();
    for (int s : id_list(d, "eos_token_id")) stops.arr.push_back(Json::make_int(s));
    spec.set("stop_ids", std::move(stops));
    return spec;
}

// The native registry of architectures: architectures[0] of a config.json -> its spec.
inline Json spec_for_config(const Json& cfg) {
    const Json* a = cfg.find("architectures");
    if (!a || a->kind != Json::Arr || a->arr.empty() || a->arr[0].kind != Json::Str)
        throw Error("config.json: key 'architectures' must be a non-empty list of names");
    if (a->arr[0].str == "Gemma2ForCausalLM") return gemma2_spec(cfg);
    throw Error("unknown architecture '" + a->arr[0].str + "' for the native host; known: Gemma2ForCausalLM "
                "(for others, hand over the spec that the Python side makes)");
}

// Stop ids of a model folder: those of generation_config.json and of config.json together
// (the reference's server reads both, runtime/src/bin/serve.rs:83-104).
inline void add_generation_stop_ids(const std::string& folder, Json& spec) {
    const std::string p = folder + "/generation_config.json";
    if (!file_exists(p)) return;
    Json g = Json::parse(read_text(p));
    std::set<int> ids;
    for (int s : cfgkey::id_list(g, "eos_token_id")) ids.insert(s);
    if (const Json* st = spec.find("stop_ids"))
        for (auto& v : st->arr) ids.insert((int)v.i);
    Json stops = Json::make_arr();
    for (int s : ids) stops.arr.push_back(Json::make_int(s));
    spec.set("stop_ids", std::move(stops));
}

}  // namespace tb

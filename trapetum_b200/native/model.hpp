// Layers put together from parts, natively: norm, position encoding, mixer (attention), feed-forward, block,
// embedding and head, each built from a spec {"kind", "params"} by a registry, none knowing which model it is
// in.  A model is a spec (the same one the Python side makes from config.json) turned into such parts, the
// tensors they declare, and the schedule in which its layers run.  Formulas in the order the reference computes
// them: runtime/src/lib.rs:4527-4540 (the sandwich of norms), :4483-4496 (attention), :4511-4516 (feed-forward),
// :4553-4561 (one forward pass); runtime/cuda/codebook_gemv.cu:192-202, 219-230, 240-270, 531-537 (the kernels).
#pragma once
#include <functional>

#include "cache.hpp"
#include "plugin.h"
#include "weights.hpp"

namespace tb {

struct PartSpec {
    std::string kind;
    Json params;
    static bool looks_like(const Json& j) { return j.kind == Json::Obj && j.has("kind") && j.has("params"); }
    static PartSpec from(const Json& j, const std::string& what) {
        if (!looks_like(j)) throw Error(what + " must be a part spec {kind, params}");
        return PartSpec{j.at("kind").string("kind"), j.at("params")};
    }
    double num(const std::string& k) const { return params.at(k).number(kind + "." + k); }
    long long integer(const std::string& k) const { return params.at(k).integer(kind + "." + k); }
    std::string str(const std::string& k) const { return params.at(k).string(kind + "." + k); }
    bool truthy(const std::string& k) const { const Json* v = params.find(k); return v && v->truthy(); }
    double num_or(const std::string& k, double d) const { return truthy(k) ? num(k) : d; }
};

struct Runtime { DType dt = BF16; };

class Part {
public:
    virtual ~Part() {}
    virtual void tensor_specs(WantedTensors&) const {}
    virtual void bind(const TensorMap&, Ops&) {}
    virtual bool graph_safe() const { return true; }
};

inline Mat tensor_of(const TensorMap& t, const std::string& name) {
    auto it = t.find(name);
    if (it == t.end()) throw Error("tensor '" + name + "' was not loaded");
    return it->second->mat();
}

// ---- norm ----------------------------------------------------------------------------------------------------
class NormPart : public Part {
public:
    virtual Mat apply(Ops& ops, const Mat& x, DType out_dt) = 0;
    // h += self(a) in place; if `then` is given, also returns then(h).  The default composes the two.
    virtual Mat add_to(Ops& ops, const Mat& h, const Partials& a, NormPart* then, DType out_dt) {
        Mat s = ops.sum_partials(a);
        Mat n = apply(ops, s, F32);
        Partials p;
        p.p = (float*)n.p; p.rows = n.rows; p.cols = n.cols; p.split_stride = n.rows * n.cols;
        ops.residual_add(h, p);
        return then ? then->apply(ops, h, out_dt) : Mat();
    }
};

// y = x * rsqrt(mean(x^2) + eps) * (offset + w); unit_offset selects the (1 + w) form
class RMSNorm : public NormPart {
public:
    RMSNorm(const PartSpec& s, const std::string& prefix, Runtime)
        : name_(prefix + s.str("weight")), size_((int)s.integer("size")), eps_((float)s.num("eps")),
          offset_(s.truthy("unit_offset") ? 1.f : 0.f) {}
    void tensor_specs(WantedTensors& w) const override { w.add(name_, TensorSpec{{size_}, "norm", false}); }
    void bind(const TensorMap& t, Ops&) override { w_ = tensor_of(t, name_); }
    Mat apply(Ops& ops, const Mat& x, DType out_dt) override { return ops.rmsnorm(x, w_, eps_, offset_, out_dt); }
    Mat add_to(Ops& ops, const Mat& h, const Partials& a, NormPart* then, DType out_dt) override {
        if (!then) return ops.add_rmsnorm(h, a, w_, eps_, offset_, nullptr, 0.f, 0.f, out_dt);
        if (auto* r = dynamic_cast<RMSNorm*>(then))
            if (r->w_.dt == w_.dt) return ops.add_rmsnorm(h, a, w_, eps_, offset_, &r->w_, r->eps_, r->offset_, out_dt);
        ops.add_rmsnorm(h, a, w_, eps_, offset_, nullptr, 0.f, 0.f, out_dt);
        return then->apply(ops, h, out_dt);
    }

private:
    std::string name_;
    int size_;
    float eps_, offset_;
    Mat w_;
};

// ---- position encoding ---------------------------------------------------------------------------------------
class PositionPart : public Part {
public:
    // true if this encoding is the rotate-half rotation of the first rotary_dim dims by position * inv_freq[i]
    // (inv_freq null: it changes nothing), so that a mixer's kernel may apply it itself
    virtual bool rotary_table(const float*& inv_freq, int& rotary_dim) const { return false; }
    virtual void rotate_and_store(Ops& ops, const Mat& qkv, int n_heads, int n_kv_heads, const StepCtx& ctx, const CacheLine& line,
                                  bool store, const Partials* partial) = 0;
};

class Rope : public PositionPart {
public:
    Rope(const PartSpec& s, const std::string&, Runtime)
        : head_dim_((int)s.integer("head_dim")), rotary_dim_(s.params.has("rotary_dim") ? (int)s.integer("rotary_dim") : head_dim_),
          theta_(s.num("theta")) {
        if (rotary_dim_ % 2 || rotary_dim_ <= 0 || rotary_dim_ > head_dim_)
            throw Error(fmt("rope: rotary_dim %d must be even and within head_dim %d", rotary_dim_, head_dim_));
        if (const Json* t = s.params.find("inv_freq")) {
            for (auto& v : t->arr) given_.push_back((float)v.number("inv_freq"));
            if ((int)given_.size() != rotary_dim_ / 2) throw Error("rope: 'inv_freq' must have rotary_dim / 2 entries");
        }
    }
    void bind(const TensorMap&, Ops&) override {
        // the table of inverse frequencies, made once in 32-bit (model/export_gemma.py:53); a spec may bring the
        // table itself ("inv_freq"), so that two hosts of one process use the same bits
        std::vector<float> f(rotary_dim_ / 2);
        for (int i = 0; i < rotary_dim_ / 2; i++) {
            const float e = (float)(2 * i) / (float)rotary_dim_;
            f[i] = given_.empty() ? 1.0f / powf((float)theta_, e) : given_[i];
        }
        inv_freq_.alloc(f.size() * 4);
        cuda_ok(cudaMemcpy(inv_freq_.p, f.data(), f.size() * 4, cudaMemcpyHostToDevice), "rope table");
    }
    bool rotary_table(const float*& inv_freq, int& rotary_dim) const override {
        inv_freq = (const float*)inv_freq_.p; rotary_dim = rotary_dim_;
        return true;
    }
    void rotate_and_store(Ops& ops, const Mat& qkv, int n_heads, int n_kv_heads, const StepCtx& ctx, const CacheLine& line,
                          bool store, const Partials* partial) override {
        ops.rope_kv(qkv, n_heads, n_kv_heads, head_dim_, rotary_dim_, (const float*)inv_freq_.p, ctx, store ? &line : nullptr, partial);
    }

private:
    int head_dim_, rotary_dim_;
    double theta_;
    std::vector<float> given_;
    DeviceBuffer inv_freq_;
};

class NoPosition : public PositionPart {
public:
    NoPosition(const PartSpec& s, const std::string&, Runtime) : head_dim_((int)s.integer("head_dim")) {}
    bool rotary_table(const float*& inv_freq, int& rotary_dim) const override { inv_freq = nullptr; rotary_dim = 0; return true; }
    void rotate_and_store(Ops& ops, const Mat& qkv, int n_heads, int n_kv_heads, const StepCtx& ctx, const CacheLine& line,
                          bool store, const Partials* partial) override {
        if (store || partial) ops.rope_kv(qkv, n_heads, n_kv_heads, head_dim_, 0, nullptr, ctx, store ? &line : nullptr, partial);
    }

private:
    int head_dim_;
};

// ---- mixer, feed-forward, block --------------------------------------------------------------------------------
class MixerPart : public Part {
public:
    virtual CacheNeed cache_need() const { return CacheNeed(); }
    // x [tokens, hidden] in the compute dtype -> the branch output as 32-bit partial sums (splits may be 1)
    virtual Partials forward(Ops& ops, const Mat& x, StepCtx& ctx, const CacheLine& line) = 0;
};

class FeedForwardPart : public Part {
public:
    virtual Partials forward(Ops& ops, const Mat& x, StepCtx& ctx) = 0;
};

// The residual stream of a step: a 32-bit [tokens, hidden] matrix and the one branch output that still waits to be
// added.  An addition is held back until the next read so that "h += norm_a(a); x = norm_b(h)" runs as one kernel,
// also across the border between two layers.
class Stream {
public:
    explicit Stream(Mat h) : h_(h) {}
    void add(const Partials& a) { flush(); pending_ = true; a_ = a; norm_ = nullptr; }
    void add_normed(const Partials& a, NormPart* n) { flush(); pending_ = true; a_ = a; norm_ = n; }
    Mat normed(Ops& ops, NormPart* n, DType out_dt) {
        ops_ = &ops;
        if (pending_) {
            pending_ = false;
            if (norm_) return norm_->add_to(ops, h_, a_, n, out_dt);
            ops.residual_add(h_, a_);
        }
        return n->apply(ops, h_, out_dt);
    }
    Mat value(Ops& ops) { ops_ = &ops; flush(); return h_; }

private:
    void flush() {
        if (!pending_) return;
        pending_ = false;
        if (norm_) norm_->add_to(*ops_, h_, a_, nullptr, F32);
        else ops_->residual_add(h_, a_);
    }
    Mat h_;
    bool pending_ = false;
    Partials a_;
    NormPart* norm_ = nullptr;
    Ops* ops_ = nullptr;
};

class BlockPart : public Part {
public:
    std::unique_ptr<MixerPart> mixer;
    std::unique_ptr<FeedForwardPart> feed_forward;
    virtual void forward(Ops& ops, Stream& stream, StepCtx& ctx, const CacheLine& line) = 0;
    bool graph_safe() const override { return mixer->graph_safe() && feed_forward->graph_safe(); }
};

// ---- registries: family and kind -> factory ----------------------------------------------------------------------
template <typename Base> struct Registry {
    typedef std::function<std::unique_ptr<Base>(const PartSpec&, const std::string& prefix, Runtime)> Factory;
    static std::map<std::string, Factory>& table() {
        static std::map<std::string, Factory> t;
        return t;
    }
    static void add(const std::string& kind, Factory f) { table()[kind] = std::move(f); }
    static bool knows(const std::string& kind) { return table().count(kind) != 0; }
    static std::unique_ptr<Base> build(const char* family, const PartSpec& s, const std::string& prefix, Runtime rt) {
        auto it = table().find(s.kind);
        if (it == table().end()) {
            std::string known;
            for (auto& kv : table()) known += (known.empty() ? "" : ", ") + kv.first;
            throw Error(std::string("no native ") + family + " of kind '" + s.kind + "' is registered (known: " + known + ")");
        }
        return it->second(s, prefix, rt);
    }
};
void register_builtin_parts();           // idempotent

// ---- attention -------------------------------------------------------------------------------------------------
// Grouped-query attention, causal, optionally windowed and soft-capped; q, k, v projections fused into one matrix
// when the weights are bound.  Query head h reads kv head h / (heads / kv_heads) (codebook_gemv.cu:244).
class Attention : public MixerPart {
public:
    Attention(const PartSpec& s, const std::string& prefix, Runtime rt)
        : prefix_(prefix), rt_(rt), hidden_((int)s.integer("hidden_size")), n_heads_((int)s.integer("num_heads")),
          n_kv_((int)s.integer("num_kv_heads")), hd_((int)s.integer("head_dim")), scale_((float)s.num("scale")),
          cap_((float)s.num_or("softcap", 0.0)), window_(s.truthy("window") ? (int)s.integer("window") : 0) {
        if (n_kv_ <= 0 || n_heads_ % n_kv_) throw Error(fmt("attention: %d heads cannot share %d kv heads", n_heads_, n_kv_));
        for (const char* k : {"q", "k", "v", "o"}) names_[k] = prefix + s.str(k);
        position_ = Registry<PositionPart>::build("position", PartSpec::from(s.params.at("position"), "attention.position"), prefix, rt);
        if (const Json* b = s.params.find("bias"))
            if (b->truthy())
                for (auto& kv : b->obj) {
                    if (kv.first != "q" && kv.first != "k" && kv.first != "v" && kv.first != "o")
                        throw Error("attention: 'bias' names '" + kv.first + "'; it knows q, k, v and o");
                    bias_names_[kv.first] = prefix + kv.second.string("bias name");
                }
        if (s.truthy("q_norm")) q_norm_ = Registry<NormPart>::build("norm", PartSpec::from(s.params.at("q_norm"), "attention.q_norm"), prefix, rt);
        if (s.truthy("k_norm")) k_norm_ = Registry<NormPart>::build("norm", PartSpec::from(s.params.at("k_norm"), "attention.k_norm"), prefix, rt);
        qd_ = n_heads_ * hd_;
        kvd_ = n_kv_ * hd_;
    }
    void tensor_specs(WantedTensors& w) const override {
        w.add(names_.at("q"), TensorSpec{{qd_, hidden_}});
        w.add(names_.at("k"), TensorSpec{{kvd_, hidden_}});
        w.add(names_.at("v"), TensorSpec{{kvd_, hidden_}});
        w.add(names_.at("o"), TensorSpec{{hidden_, qd_}});
        for (auto& kv : bias_names_)
            w.add(kv.second, TensorSpec{{kv.first == "q" ? qd_ : kv.first == "o" ? hidden_ : kvd_}});
        if (q_norm_) q_norm_->tensor_specs(w);
        if (k_norm_) k_norm_->tensor_specs(w);
    }
    void bind(const TensorMap& t, Ops& ops) override {
        Mat q = tensor_of(t, names_["q"]), k = tensor_of(t, names_["k"]), v = tensor_of(t, names_["v"]);
        if (q.dt != k.dt || q.dt != v.dt) throw Error("attention: q, k and v weights must be stored in one dtype");
        const int64_t width = qd_ + 2 * kvd_;
        w_qkv_buf_.alloc((size_t)width * hidden_ * dtype_size(q.dt));
        w_qkv_ = Mat(w_qkv_buf_.p, q.dt, width, hidden_);
        cuda_ok(cudaMemcpy(w_qkv_.at(0), q.p, q.bytes(), cudaMemcpyDeviceToDevice), "fusing q, k, v");
        cuda_ok(cudaMemcpy(w_qkv_.at(qd_), k.p, k.bytes(), cudaMemcpyDeviceToDevice), "fusing q, k, v");
        cuda_ok(cudaMemcpy(w_qkv_.at(qd_ + kvd_), v.p, v.bytes(), cudaMemcpyDeviceToDevice), "fusing q, k, v");
        w_o_ = tensor_of(t, names_["o"]);
        keep_ = t.at(names_["o"]);
        position_->bind(t, ops);
        if (bias_names_.count("q") || bias_names_.count("k") || bias_names_.count("v")) {
            // one 32-bit bias row for the fused projection; a projection without a bias of its own gets zeros
            std::vector<float> row((size_t)width, 0.f);
            size_t off = 0;
            for (auto& part : {std::make_pair("q", qd_), std::make_pair("k", kvd_), std::make_pair("v", kvd_)}) {
                if (bias_names_.count(part.first)) download_float(tensor_of(t, bias_names_[part.first]), row.data() + off);
                off += part.second;
            }
            b_qkv_buf_.alloc(row.size() * 4);
            cuda_ok(cudaMemcpy(b_qkv_buf_.p, row.data(), row.size() * 4, cudaMemcpyHostToDevice), "bias");
            b_qkv_ = Mat(b_qkv_buf_.p, F32, 1, width);
        }
        if (bias_names_.count("o")) {
            std::vector<float> row((size_t)hidden_);
            download_float(tensor_of(t, bias_names_["o"]), row.data());
            b_o_buf_.alloc(row.size() * 4);
            cuda_ok(cudaMemcpy(b_o_buf_.p, row.data(), row.size() * 4, cudaMemcpyHostToDevice), "bias");
            b_o_ = Mat(b_o_buf_.p, F32, 1, hidden_);
        }
        if (q_norm_) q_norm_->bind(t, ops);
        if (k_norm_) k_norm_->bind(t, ops);
    }
    CacheNeed cache_need() const override {
        CacheNeed n;
        n.kind = CacheNeed::KV; n.n_kv_heads = n_kv_; n.head_dim = hd_; n.window = window_;
        return n;
    }
    // whether this mixer is what the decode kernel's own prologue computes: the plain projection, then a
    // rotate-half rotation (or none)
    bool fused_decode() const {
        const float* f; int r;
        return !b_qkv_ && !q_norm_ && !k_norm_ && position_->rotary_table(f, r);
    }
    Partials forward(Ops& ops, const Mat& x, StepCtx& ctx, const CacheLine& line) override {
        const DType dt = rt_.dt;
        Mat q, k, v;
        if (line.owner) {
            const bool plain = !b_qkv_ && !q_norm_ && !k_norm_;
            Mat qkv;
            // keys and values that a later call of this step reads must outlive this layer's scratch
            const Arena::Region region = ops.arena->current();
            if (ctx.is_prefill && line.shared) ops.arena->use(Arena::STEP);
            if (plain && dt == BF16 && x.rows <= 128 && Ops::gemm_tc_takes(x, w_qkv_)) {
                // few tokens: the product comes as split-K partial sums, which the rotation kernel adds up
                Partials part = ops.gemm_tc_partials(x, w_qkv_);
                const float* inv_freq = nullptr;
                int rotary_dim = 0;
                if (!ctx.is_prefill && fused_decode() && Ops::attn_decode_rotates(dt, n_heads_, n_kv_, hd_)) {
                    // decoding: the attention kernel adds them up, rotates and appends to the cache by itself
                    position_->rotary_table(inv_freq, rotary_dim);
                    Mat o = ops.attn_decode(nullptr, &part, inv_freq, rotary_dim, line, ctx, n_heads_, n_kv_, hd_, scale_, cap_, window_);
                    return out(ops, o);
                }
                qkv = ops.arena->mat(dt, part.rows, part.cols);
                position_->rotate_and_store(ops, qkv, n_heads_, n_kv_, ctx, line, true, &part);
            } else {
                qkv = ops.linear(x, w_qkv_, dt);
                finish_projection(ops, qkv, n_heads_, n_kv_);
                position_->rotate_and_store(ops, qkv, n_heads_, n_kv_, ctx, line, true, nullptr);
            }
            ops.arena->use(region);
            q = qkv.cols_slice(0, qd_);
            k = qkv.cols_slice(qd_, kvd_);
            v = qkv.cols_slice(qd_ + kvd_, kvd_);
            if (ctx.is_prefill && line.shared) ctx.step_kv[line.entry] = {k, v};      // a later call that reads this cache needs them
        } else {
            // this call reads another call's cache: only its queries are new
            q = ops.linear(x, w_qkv_.rows_slice(0, qd_), dt);
            finish_projection(ops, q, n_heads_, 0);
            position_->rotate_and_store(ops, q, n_heads_, 0, ctx, line, false, nullptr);
            if (ctx.is_prefill) { k = ctx.step_kv.at(line.entry).first; v = ctx.step_kv.at(line.entry).second; }
        }
        Mat o = ctx.is_prefill ? ops.attn_prefill(q, k, v, ctx, n_heads_, n_kv_, hd_, scale_, cap_, window_)
                               : ops.attn_decode(&q, nullptr, nullptr, 0, line, ctx, n_heads_, n_kv_, hd_, scale_, cap_, window_);
        return out(ops, o);
    }

private:
    static void download_float(const Mat& m, float* dst) {
        const int64_t n = m.rows * m.cols;
        if (m.dt == F32) { cuda_ok(cudaMemcpy(dst, m.p, n * 4, cudaMemcpyDeviceToHost), "bias"); return; }
        std::vector<uint16_t> h((size_t)n);
        cuda_ok(cudaMemcpy(h.data(), m.p, n * 2, cudaMemcpyDeviceToHost), "bias");
        for (int64_t i = 0; i < n; i++) { uint32_t u = (uint32_t)h[i] << 16; memcpy(dst + i, &u, 4); }
    }
    // bias and head norms on a freshly projected [tokens, (n_q + 2 n_kv) * head_dim] matrix, in place
    void finish_projection(Ops& ops, const Mat& qkv, int n_q, int n_kv) {
        if (b_qkv_) ops.add_bias(qkv, b_qkv_.cols_slice(0, qkv.cols));
        struct Item { NormPart* norm; int64_t lo; int n; } items[2] = {{q_norm_.get(), 0, n_q}, {k_norm_.get(), (int64_t)n_q * hd_, n_kv}};
        for (auto& it : items) {
            if (!it.norm || !it.n) continue;
            // the heads of all tokens as rows of a contiguous [tokens * heads, head_dim] matrix, normed, written back
            const int64_t T = qkv.rows, w = (int64_t)it.n * hd_;
            Mat heads = ops.arena->mat(qkv.dt, T * it.n, hd_);
            const size_t es = dtype_size(qkv.dt);
            if (!ops.dry())
                cuda_ok(cudaMemcpy2DAsync(heads.p, w * es, qkv.at(0, it.lo), qkv.ld * es, w * es, T, cudaMemcpyDeviceToDevice, ops.stream), "head norm");
            Mat normed = it.norm->apply(ops, heads, qkv.dt);
            if (!ops.dry())
                cuda_ok(cudaMemcpy2DAsync(qkv.at(0, it.lo), qkv.ld * es, normed.p, w * es, w * es, T, cudaMemcpyDeviceToDevice, ops.stream), "head norm");
        }
    }
    Partials out(Ops& ops, const Mat& o) {
        Partials p = ops.linear_partials(o, w_o_);
        if (b_o_) ops.add_bias(p.first(), b_o_);
        return p;
    }
    std::string prefix_;
    Runtime rt_;
    int hidden_, n_heads_, n_kv_, hd_;
    float scale_, cap_;
    int window_;
    int64_t qd_ = 0, kvd_ = 0;
    std::map<std::string, std::string> names_, bias_names_;
    std::unique_ptr<PositionPart> position_;
    std::unique_ptr<NormPart> q_norm_, k_norm_;
    DeviceBuffer w_qkv_buf_, b_qkv_buf_, b_o_buf_;
    Mat w_qkv_, w_o_, b_qkv_, b_o_;
    std::shared_ptr<DeviceTensor> keep_;
};

// ---- parts from outside the library (plugin.h): a mixer or a feed-forward described by a table of functions -----------
class PluginCore {
public:
    PluginCore(const char* what, const tb_mixer_plugin* p, const PartSpec& s, const std::string& prefix, Runtime rt)
        : p_(p), what_(std::string(what) + " '" + s.kind + "'") {
        const char* err = nullptr;
        self_ = p->create(s.params.dump().c_str(), prefix.c_str(), (int)rt.dt, &err);
        if (!self_) throw Error(what_ + " could not be made: " + (err ? err : "no reason given"));
    }
    ~PluginCore() {
        if (self_ && p_->destroy) p_->destroy(self_);
    }
    PluginCore(const PluginCore&) = delete;
    PluginCore& operator=(const PluginCore&) = delete;

    void tensor_specs(WantedTensors& w) const {
        const int n = p_->tensor_count ? p_->tensor_count(self_) : 0;
        for (int i = 0; i < n; i++) {
            tb_tensor_decl d;
            memset(&d, 0, sizeof d);
            if (p_->tensor_decl(self_, i, &d)) throw Error(what_ + ": tensor_decl failed");
            TensorSpec ts;
            ts.shape.assign(d.shape, d.shape + d.ndim);
            ts.role = d.role[0] ? d.role : "matrix";
            ts.optional = d.optional != 0;
            w.add(d.name, ts);
        }
    }
    void bind(const TensorMap& t) {
        const int n = p_->tensor_count ? p_->tensor_count(self_) : 0;
        for (int i = 0; i < n; i++) {
            tb_tensor_decl d;
            memset(&d, 0, sizeof d);
            p_->tensor_decl(self_, i, &d);
            auto it = t.find(d.name);
            if (it == t.end()) continue;
            keep_.push_back(it->second);
            const char* err = nullptr;
            if (p_->bind(self_, d.name, it->second->buf.p, (int)it->second->dt, &err))
                throw Error(what_ + " refused tensor " + d.name + ": " + (err ? err : "no reason given"));
        }
    }
    bool graph_safe() const { return p_->graph_safe != 0; }
    CacheNeed cache_need() const {
        CacheNeed n;
        tb_cache_need c;
        memset(&c, 0, sizeof c);
        if (p_->cache_need && p_->cache_need(self_, &c)) throw Error(what_ + ": cache_need failed");
        n.kind = c.kind == TB_NEED_KV ? CacheNeed::KV : c.kind == TB_NEED_STATE ? CacheNeed::STATE : CacheNeed::NONE;
        n.n_kv_heads = c.n_kv_heads; n.head_dim = c.head_dim; n.window = c.window; n.state_bytes = (size_t)c.state_bytes;
        return n;
    }
    // line: the mixer's cache line; a feed-forward has none
    Partials forward(Ops& ops, const Mat& x, StepCtx& ctx, const CacheLine* line) {
        Mat out = ops.arena->mat(F32, x.rows, x.cols);
        tb_part_ctx c;
        memset(&c, 0, sizeof c);
        c.stream = ops.stream; c.dry = ops.dry() ? 1 : 0; c.is_prefill = ctx.is_prefill; c.n_tokens = ctx.n_tokens; c.batch = ctx.batch;
        c.positions = ctx.positions; c.token_seq = ctx.token_seq; c.seq_start = ctx.seq_start; c.len_after = ctx.len_after;
        c.slot_ids = ctx.slot_ids; c.host_slots = ctx.slots.data(); c.host_seq_lens = ctx.seq_lens.data();
        if (line) {
            c.state = line->state; c.state_bytes = (long long)line->state_bytes;
            c.k = line->k; c.v = line->v; c.page_table = line->page_table; c.pt_stride = line->pt_stride; c.ring_rows = line->ring_rows;
            c.line_owner = line->owner ? 1 : 0;
        }
        c.alloc = [](void* a, size_t bytes) { return ((Arena*)a)->alloc(bytes); };
        c.arena = ops.arena;
        const char* err = nullptr;
        if (p_->forward(self_, &c, x.p, (int)x.dt, x.rows, x.cols, (float*)out.p, &err))
            throw Error(what_ + " failed: " + (err ? err : "no reason given"));
        Partials r;
        r.p = (float*)out.p; r.rows = out.rows; r.cols = out.cols; r.split_stride = out.rows * out.cols;
        return r;
    }

private:
    const tb_mixer_plugin* p_;
    void* self_ = nullptr;
    std::string what_;
    std::vector<std::shared_ptr<DeviceTensor>> keep_;
};

class PluginMixer : public MixerPart {
public:
    PluginMixer(const tb_mixer_plugin* p, const PartSpec& s, const std::string& prefix, Runtime rt) : core_("mixer", p, s, prefix, rt) {}
    void tensor_specs(WantedTensors& w) const override { core_.tensor_specs(w); }
    void bind(const TensorMap& t, Ops&) override { core_.bind(t); }
    bool graph_safe() const override { return core_.graph_safe(); }
    CacheNeed cache_need() const override { return core_.cache_need(); }
    Partials forward(Ops& ops, const Mat& x, StepCtx& ctx, const CacheLine& line) override { return core_.forward(ops, x, ctx, &line); }

private:
    PluginCore core_;
};

// The same table describes a feed-forward: it has no cache (cache_need is not asked) and gets no cache line.
class PluginFeedForward : public FeedForwardPart {
public:
    PluginFeedForward(const tb_mixer_plugin* p, const PartSpec& s, const std::string& prefix, Runtime rt)
        : core_("feed-forward", p, s, prefix, rt) {}
    void tensor_specs(WantedTensors& w) const override { core_.tensor_specs(w); }
    void bind(const TensorMap& t, Ops&) override { core_.bind(t); }
    bool graph_safe() const override { return core_.graph_safe(); }
    Partials forward(Ops& ops, const Mat& x, StepCtx& ctx) override { return core_.forward(ops, x, ctx, nullptr); }

private:
    PluginCore core_;
};

// ---- gated dense feed-forward: down(act(gate(x)) * up(x)) ---------------------------------------------------------
class GatedMLP : public FeedForwardPart {
public:
    GatedMLP(const PartSpec& s, const std::string& prefix, Runtime rt)
        : rt_(rt), hidden_((int)s.integer("hidden_size")), inter_((int)s.integer("intermediate_size")),
          act_(activation_code(s.str("activation"))), gate_(prefix + s.str("gate")), up_(prefix + s.str("up")),
          down_(prefix + s.str("down")) {}
    void tensor_specs(WantedTensors& w) const override {
        w.add(gate_, TensorSpec{{inter_, hidden_}});
        w.add(up_, TensorSpec{{inter_, hidden_}});
        w.add(down_, TensorSpec{{hidden_, inter_}});
    }
    void bind(const TensorMap& t, Ops&) override {
        Mat g = tensor_of(t, gate_), u = tensor_of(t, up_);
        if (g.dt != u.dt) throw Error("gated_mlp: gate and up weights must be stored in one dtype");
        // With bfloat16 weights of tensor-core sizes the activation runs in the product's epilogue; the gate and up
        // rows are then interleaved in blocks of 16.  Otherwise: [gate; up] and a kernel of its own.
        fused_ = g.dt == BF16 && rt_.dt == BF16 && inter_ % 16 == 0 && hidden_ % 8 == 0;
        const size_t es = dtype_size(g.dt), row = (size_t)hidden_ * es;
        w_gu_buf_.alloc(2 * (size_t)inter_ * row);
        w_gu_ = Mat(w_gu_buf_.p, g.dt, 2 * (int64_t)inter_, hidden_);
        if (fused_) {
            cuda_ok(cudaMemcpy2D(w_gu_.p, 32 * row, g.p, 16 * row, 16 * row, inter_ / 16, cudaMemcpyDeviceToDevice), "interleaving gate and up");
            cuda_ok(cudaMemcpy2D((char*)w_gu_.p + 16 * row, 32 * row, u.p, 16 * row, 16 * row, inter_ / 16, cudaMemcpyDeviceToDevice),
                    "interleaving gate and up");
        } else {
            cuda_ok(cudaMemcpy(w_gu_.p, g.p, g.bytes(), cudaMemcpyDeviceToDevice), "fusing gate and up");
            cuda_ok(cudaMemcpy(w_gu_.at(inter_), u.p, u.bytes(), cudaMemcpyDeviceToDevice), "fusing gate and up");
        }
        w_down_ = tensor_of(t, down_);
        keep_ = t.at(down_);
    }
    Partials forward(Ops& ops, const Mat& x, StepCtx&) override {
        if (fused_) {
            Ops::need(Ops::gemm_tc_takes(x, w_gu_), "gated_mlp: the interleaved weights need the tensor-core product, which does not take this input");
            Mat act = ops.gemm_tc_gated(x, w_gu_, act_);
            return ops.linear_partials(act, w_down_);
        }
        Mat gu = ops.linear(x, w_gu_, rt_.dt);
        Mat act = ops.gated_act(gu, act_, rt_.dt);
        return ops.linear_partials(act, w_down_);
    }

private:
    Runtime rt_;
    int hidden_, inter_, act_;
    std::string gate_, up_, down_;
    bool fused_ = false;
    DeviceBuffer w_gu_buf_;
    Mat w_gu_, w_down_;
    std::shared_ptr<DeviceTensor> keep_;
};

// ---- blocks ----------------------------------------------------------------------------------------------------
class NormedBlock : public BlockPart {
public:
    NormedBlock(const PartSpec& s, const std::string& prefix, Runtime rt, std::vector<std::string> names) : rt_(rt) {
        for (auto& n : names) norms_[n] = Registry<NormPart>::build("norm", PartSpec::from(s.params.at(n), "block." + n), prefix, rt);
    }
    void tensor_specs(WantedTensors& w) const override {
        for (auto& kv : norms_) kv.second->tensor_specs(w);
        mixer->tensor_specs(w);
        feed_forward->tensor_specs(w);
    }
    void bind(const TensorMap& t, Ops& ops) override {
        for (auto& kv : norms_) kv.second->bind(t, ops);
        mixer->bind(t, ops);
        feed_forward->bind(t, ops);
    }

protected:
    Runtime rt_;
    std::map<std::string, std::unique_ptr<NormPart>> norms_;
};

// h += post_mixer_norm(mixer(pre_mixer_norm(h))); h += post_ffn_norm(feed_forward(pre_ffn_norm(h)))   (lib.rs:4527-4540)
class SandwichBlock : public NormedBlock {
public:
    SandwichBlock(const PartSpec& s, const std::string& prefix, Runtime rt)
        : NormedBlock(s, prefix, rt, {"pre_mixer_norm", "post_mixer_norm", "pre_ffn_norm", "post_ffn_norm"}) {}
    void forward(Ops& ops, Stream& stream, StepCtx& ctx, const CacheLine& line) override {
        Mat x = stream.normed(ops, norms_["pre_mixer_norm"].get(), rt_.dt);
        stream.add_normed(mixer->forward(ops, x, ctx, line), norms_["post_mixer_norm"].get());
        x = stream.normed(ops, norms_["pre_ffn_norm"].get(), rt_.dt);
        stream.add_normed(feed_forward->forward(ops, x, ctx), norms_["post_ffn_norm"].get());
    }
};

// h += mixer(pre_mixer_norm(h)); h += feed_forward(pre_ffn_norm(h))
class PreNormBlock : public NormedBlock {
public:
    PreNormBlock(const PartSpec& s, const std::string& prefix, Runtime rt) : NormedBlock(s, prefix, rt, {"pre_mixer_norm", "pre_ffn_norm"}) {}
    void forward(Ops& ops, Stream& stream, StepCtx& ctx, const CacheLine& line) override {
        Mat x = stream.normed(ops, norms_["pre_mixer_norm"].get(), rt_.dt);
        stream.add(mixer->forward(ops, x, ctx, line));
        x = stream.normed(ops, norms_["pre_ffn_norm"].get(), rt_.dt);
        stream.add(feed_forward->forward(ops, x, ctx));
    }
};

inline void register_builtin_parts() {
    static bool done = false;
    if (done) return;
    done = true;
    Registry<NormPart>::add("rmsnorm", [](const PartSpec& s, const std::string& p, Runtime rt) { return std::unique_ptr<NormPart>(new RMSNorm(s, p, rt)); });
    Registry<PositionPart>::add("rope", [](const PartSpec& s, const std::string& p, Runtime rt) { return std::unique_ptr<PositionPart>(new Rope(s, p, rt)); });
    Registry<PositionPart>::add("none", [](const PartSpec& s, const std::string& p, Runtime rt) { return std::unique_ptr<PositionPart>(new NoPosition(s, p, rt)); });
    Registry<MixerPart>::add("attention", [](const PartSpec& s, const std::string& p, Runtime rt) { return std::unique_ptr<MixerPart>(new Attention(s, p, rt)); });
    Registry<FeedForwardPart>::add("gated_mlp", [](const PartSpec& s, const std::string& p, Runtime rt) { return std::unique_ptr<FeedForwardPart>(new GatedMLP(s, p, rt)); });
    Registry<BlockPart>::add("sandwich", [](const PartSpec& s, const std::string& p, Runtime rt) { return std::unique_ptr<BlockPart>(new SandwichBlock(s, p, rt)); });
    Registry<BlockPart>::add("pre_norm", [](const PartSpec& s, const std::string& p, Runtime rt) { return std::unique_ptr<BlockPart>(new PreNormBlock(s, p, rt)); });
}

// ---- the model ---------------------------------------------------------------------------------------------------
struct ScheduleEntry { int layer; int cache_of; };          // cache_of < 0: its own

class Model {
public:
    Json spec;
    Runtime rt;
    int device = 0;
    int hidden = 0, vocab = 0, max_positions = 0;
    std::vector<int> stop_ids;
    std::vector<ScheduleEntry> schedule;
    std::vector<std::unique_ptr<BlockPart>> blocks;

    // Whether every part kind that a spec names has a native class (else the model runs on the Python host).
    static bool spec_is_native(const Json& spec, std::string* why = nullptr) {
        register_builtin_parts();
        auto miss = [&](const std::string& w) { if (why) *why = w; return false; };
        try {
            if (spec.at("embedding").at("kind").str != "embedding") return miss("embedding of kind " + spec.at("embedding").at("kind").str);
            if (spec.at("head").at("kind").str != "linear_head") return miss("head of kind " + spec.at("head").at("kind").str);
            if (!Registry<NormPart>::knows(spec.at("final_norm").at("kind").str)) return miss("norm of kind " + spec.at("final_norm").at("kind").str);
            for (auto& l : spec.at("layers").arr) {
                if (!Registry<BlockPart>::knows(l.at("block").at("kind").str)) return miss("block of kind " + l.at("block").at("kind").str);
                if (!Registry<MixerPart>::knows(l.at("mixer").at("kind").str)) return miss("mixer of kind " + l.at("mixer").at("kind").str);
                if (!Registry<FeedForwardPart>::knows(l.at("feed_forward").at("kind").str))
                    return miss("feed_forward of kind " + l.at("feed_forward").at("kind").str);
                for (auto& kv : l.at("block").at("params").obj)
                    if (PartSpec::looks_like(kv.second) && !Registry<NormPart>::knows(kv.second.at("kind").str))
                        return miss("norm of kind " + kv.second.at("kind").str);
                const Json& mp = l.at("mixer").at("params");
                if (const Json* pos = mp.find("position"))
                    if (PartSpec::looks_like(*pos) && !Registry<PositionPart>::knows(pos->at("kind").str))
                        return miss("position of kind " + pos->at("kind").str);
            }
        } catch (const Error& e) {
            return miss(e.what());
        }
        return true;
    }

    Model(const Json& spec_, DType dt, int device_) : spec(spec_), device(device_) {
        register_builtin_parts();
        rt.dt = dt;
        hidden = (int)spec.at("hidden_size").integer("hidden_size");
        vocab = (int)spec.at("vocab_size").integer("vocab_size");
        max_positions = (int)spec.at("max_positions").integer("max_positions");
        if (const Json* s = spec.find("stop_ids"))
            for (auto& v : s->arr) stop_ids.push_back((int)v.integer("stop id"));
        PartSpec emb = PartSpec::from(spec.at("embedding"), "embedding");
        if (emb.kind != "embedding") throw Error("no native embedding of kind '" + emb.kind + "'");
        emb_name_ = emb.str("weight");
        emb_scale_ = (float)emb.num_or("scale", 1.0);
        emb_vocab_ = (int)emb.integer("vocab_size");
        for (auto& l : spec.at("layers").arr) {
            const std::string prefix = l.at("prefix").string("prefix");
            auto block = Registry<BlockPart>::build("block", PartSpec::from(l.at("block"), "block"), prefix, rt);
            block->mixer = Registry<MixerPart>::build("mixer", PartSpec::from(l.at("mixer"), "mixer"), prefix, rt);
            block->feed_forward = Registry<FeedForwardPart>::build("feed_forward", PartSpec::from(l.at("feed_forward"), "feed_forward"), prefix, rt);
            blocks.push_back(std::move(block));
        }
        for (auto& e : spec.at("schedule").arr) {
            ScheduleEntry s;
            s.layer = (int)e.at("layer").integer("schedule layer");
            const Json* c = e.find("cache_of");
            s.cache_of = (c && !c->is_null()) ? (int)c->integer("cache_of") : -1;
            const int idx = (int)schedule.size();
            if (s.layer < 0 || s.layer >= (int)blocks.size())
                throw Error(fmt("schedule entry %d names layer %d, but the model has %zu layers", idx, s.layer, blocks.size()));
            if (s.cache_of >= 0 && (s.cache_of >= idx || schedule[s.cache_of].cache_of >= 0))
                throw Error(fmt("schedule entry %d reads the cache of entry %d, which must be an earlier entry that owns one", idx, s.cache_of));
            schedule.push_back(s);
        }
        final_norm_ = Registry<NormPart>::build("norm", PartSpec::from(spec.at("final_norm"), "final_norm"), "", rt);
        PartSpec head = PartSpec::from(spec.at("head"), "head");
        if (head.kind != "linear_head") throw Error("no native head of kind '" + head.kind + "'");
        head_name_ = head.str("weight");
        head_cap_ = (float)head.num_or("softcap", 0.0);
        if (head.truthy("tied_to")) head_tied_ = head.str("tied_to");
        head_vocab_ = (int)head.integer("vocab_size");
    }

    WantedTensors wanted() const {
        WantedTensors w;
        w.add(emb_name_, TensorSpec{{emb_vocab_, hidden}, "embedding"});
        for (auto& b : blocks) b->tensor_specs(w);
        final_norm_->tensor_specs(w);
        w.add(head_name_, TensorSpec{{head_vocab_, hidden}, "matrix", !head_tied_.empty()});
        if (!head_tied_.empty()) w.add(head_tied_, TensorSpec{{head_vocab_, hidden}, "embedding"});
        return w;
    }
    void bind(TensorMap tensors, Ops& ops) {
        tensors_ = std::move(tensors);
        emb_ = tensor_of(tensors_, emb_name_);
        for (auto& b : blocks) b->bind(tensors_, ops);
        final_norm_->bind(tensors_, ops);
        head_ = tensors_.count(head_name_) ? tensor_of(tensors_, head_name_) : tensor_of(tensors_, head_tied_);
        // the separate q, k, v, gate and up matrices were copied into fused ones: let them go
        for (auto& l : spec.at("layers").arr) {
            const std::string prefix = l.at("prefix").str;
            for (const char* family : {"mixer", "feed_forward"}) {
                const Json& p = l.at(family).at("params");
                for (const char* k : {"q", "k", "v", "gate", "up"})
                    if (const Json* n = p.find(k))
                        if (n->kind == Json::Str) tensors_.erase(prefix + n->str);
            }
        }
        cuda_ok(cudaDeviceSynchronize(), "binding weights");
    }
    bool graph_safe() const {
        for (auto& b : blocks) if (!b->graph_safe()) return false;
        return true;
    }
    // (owning entry -> need, entries whose cache someone else reads)
    void cache_needs(std::map<int, CacheNeed>& needs, std::set<int>& shared) const {
        for (size_t e = 0; e < schedule.size(); e++) {
            if (schedule[e].cache_of < 0) needs[(int)e] = blocks[schedule[e].layer]->mixer->cache_need();
            else shared.insert(schedule[e].cache_of);
        }
    }

    // ids int32 [tokens] on the device -> float32 logits [wanted rows, vocab] (all rows if want_rows is null).
    // n_want 0 with want_rows set: the layers run (they fill the cache), the head does not.
    Mat forward(Ops& ops, const int* ids, StepCtx& ctx, Cache& cache, const std::vector<CacheLine>& lines, const int* want_rows, int n_want) {
        Arena& ar = *ops.arena;
        ar.use(Arena::STEP);
        Stream stream(ops.embed(ids, emb_, emb_scale_, ctx.n_tokens));
        for (size_t e = 0; e < schedule.size(); e++) {
            const Arena::Region r = (e & 1) ? Arena::LAYER_B : Arena::LAYER_A;
            ar.reset(r);
            ar.use(r);
            blocks[schedule[e].layer]->forward(ops, stream, ctx, lines[e]);
        }
        ar.use(Arena::STEP);
        Mat h = stream.value(ops);
        if (want_rows) {
            if (n_want == 0) return Mat();
            h = ops.gather_rows(h, want_rows, n_want);
        }
        Mat x = final_norm_->apply(ops, h, rt.dt);
        return ops.linear(x, head_, F32, head_cap_);
    }

private:
    std::string emb_name_, head_name_, head_tied_;
    float emb_scale_ = 1.f, head_cap_ = 0.f;
    int emb_vocab_ = 0, head_vocab_ = 0;
    Mat emb_, head_;
    std::unique_ptr<NormPart> final_norm_;
    TensorMap tensors_;
};

}  // namespace tb

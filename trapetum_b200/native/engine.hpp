// The engine: a model, its cache, and the step function over both; and the generation loop above it.
//
// A batch is a set of sequences that start together.  Its first step brings every sequence's whole prompt
// (lengths may differ; tokens are packed back to back, no padding exists anywhere); every later step brings
// exactly one token for each sequence that is still alive.  A step runs only the tokens it is given, on top of
// the cache the earlier steps left, and returns the logits at the places asked for.  Decode steps of one
// (batch size, length bucket, even/uneven lengths) are captured into a CUDA graph on their second occurrence.
// The reference's forward takes one token of one sequence (runtime/src/lib.rs:4553-4561), so a prompt costs one
// call per token (runtime/src/bin/gemma_run.rs:12), and its loop is one greedy sequence (:12-15).
#pragma once
#include <deque>

#include "gemma2.hpp"

namespace tb {

struct StepError : Error {
    using Error::Error;
};

// How much a batch's context lengths differ, in quarters: 0 if their sum is at least three quarters of
// batch x longest, 1 from a half on, 2 from a quarter on, else 3 (what share of the GPU stays idle if work is dealt
// out by the longest sequence).  Launch shapes depend on the lengths only through this and the bucket.
inline int unevenness(const std::vector<int>& lens) {
    if (lens.size() <= 1) return 0;
    long long sum = 0;
    int mx = 0;
    for (int l : lens) { sum += l; mx = std::max(mx, l); }
    const long long full = (long long)lens.size() * mx;
    if (full <= 0) return 0;
    const long long q = (4 * sum) / full;                        // quarters that are filled, rounded down (0..4)
    return (int)std::max(0LL, std::min(3LL, 3 - q));
}

inline int len_bucket(int max_len) {
    int b = 256;
    while (b < max_len) b *= 2;
    return b;
}

// A pinned host buffer and its device twin for a step's integer inputs: one copy per step.
struct InputBuffer {
    int* host = nullptr;
    DeviceBuffer dev;
    size_t cap = 0;
    cudaEvent_t copied = nullptr;
    bool pending = false;
    ~InputBuffer() {
        if (host) cudaFreeHost(host);
        if (copied) cudaEventDestroy(copied);
    }
    void reserve(size_t ints) {
        if (ints <= cap) return;
        wait();
        if (host) cudaFreeHost(host);
        cap = std::max<size_t>(1024, ints * 2);
        cuda_ok(cudaMallocHost((void**)&host, cap * 4), "pinned input buffer");
        dev.alloc(cap * 4);
        if (!copied) cuda_ok(cudaEventCreateWithFlags(&copied, cudaEventDisableTiming), "event");
    }
    void wait() {
        if (pending) { cuda_ok(cudaEventSynchronize(copied), "waiting for the last input copy"); pending = false; }
    }
    void upload(size_t ints, cudaStream_t s) {
        cuda_ok(cudaMemcpyAsync(dev.p, host, ints * 4, cudaMemcpyHostToDevice, s), "copying a step's inputs");
        cuda_ok(cudaEventRecord(copied, s), "event");
        pending = true;
    }
    const int* d(size_t off) const { return (const int*)dev.p + off; }
};

// The ids of a step taken from the device: row i of the step gets ids[src_rows[i]] (the greedy choice of an
// earlier step that the host has not read yet).
struct DeviceIds {
    const int* ids = nullptr;
    int n_src = 0;
    std::vector<int> src_rows;
};

struct StepResult {
    const float* logits = nullptr;       // device, [rows, vocab] (null when greedy or nothing wanted)
    const int* ids = nullptr;            // device, [rows] chosen ids (greedy steps)
    int rows = 0;
};

class Engine {
public:
    Model& model;
    std::unique_ptr<Cache> cache;
    Ops ops;
    bool use_graphs;
    long long h2d_bytes_last = 0;

    Engine(Model& m, long long max_tokens, int max_slots, bool graphs) : model(m), use_graphs(graphs) {
        cuda_ok(cudaSetDevice(m.device), "selecting the device");
        std::map<int, CacheNeed> needs;
        std::set<int> shared;
        m.cache_needs(needs, shared);
        cache.reset(new Cache(needs, shared, max_tokens, m.rt.dt, max_slots));
        cudaDeviceProp prop;
        cuda_ok(cudaGetDeviceProperties(&prop, m.device), "device properties");
        ops.sms = prop.multiProcessorCount;
        cuda_ok(cudaStreamCreateWithFlags(&own_stream_, cudaStreamNonBlocking), "stream");
        ops.stream = own_stream_;
        tickets_.alloc(Ops::TICKET_SLOTS * 4);
        cuda_ok(cudaMemset(tickets_.p, 0, Ops::TICKET_SLOTS * 4), "ticket counters");
        ops.tickets = (int*)tickets_.p;
        arena_.reserve(1 << 20, 1 << 20);
        ops.arena = &arena_;
        graph_safe_ = m.graph_safe();
    }
    ~Engine() {
        cudaStreamSynchronize(ops.stream);
        for (auto& kv : decode_) if (kv.second->exec) cudaGraphExecDestroy(kv.second->exec);
        if (own_stream_) cudaStreamDestroy(own_stream_);
    }
    // Run on a stream of the caller's (for instance the one a tensor library uses), so that its work and the
    // engine's are ordered.  Captured graphs are dropped: they replay on any stream, but their scratch is per shape.
    void set_stream(cudaStream_t s) { ops.stream = s; }
    void use_own_stream() { ops.stream = own_stream_; }
    void synchronize() { cuda_ok(cudaStreamSynchronize(ops.stream), "synchronize"); }

    std::vector<int> start(int n) {
        std::vector<int> got;
        try {
            for (int i = 0; i < n; i++) got.push_back(cache->claim(ops.stream));
        } catch (...) {
            for (int s : got) cache->release(s);
            throw;
        }
        return got;
    }
    void release(const std::vector<int>& slots) {
        for (int s : slots) cache->release(s);
    }

    // One step.  tokens[i]: the new tokens of sequence i; want[i]: the places among them whose logits are returned,
    // in the order of the sequences and of the lists (want null: each sequence's last token).  greedy: instead of
    // the logits, the ids of the largest logit at each wanted place (the smallest id on a tie).
    StepResult step(const std::vector<int>& slots, const std::vector<std::vector<int>>& tokens,
                    const std::vector<std::vector<int>>* want_in, bool greedy, const DeviceIds* chained = nullptr) {
        const bool is_prefill = classify(slots, tokens);
        const int B = (int)slots.size(), V = model.vocab;
        std::vector<int> lens(B);
        for (int i = 0; i < B; i++) {
            lens[i] = (int)tokens[i].size();
            for (int tok : tokens[i])
                if (tok < 0 || tok >= V) throw StepError(fmt("sequence %d: token id %d is outside the vocabulary [0, %d)", i, tok, V));
        }
        std::vector<std::vector<int>> want_default;
        if (!want_in) {
            for (int i = 0; i < B; i++) want_default.push_back({lens[i] - 1});
            want_in = &want_default;
        }
        const auto& want = *want_in;
        if ((int)want.size() != B) throw StepError(fmt("%d sequences but %zu 'want' lists", B, want.size()));
        for (int i = 0; i < B; i++)
            for (int j : want[i])
                if (j < 0 || j >= lens[i]) throw StepError(fmt("sequence %d: wanted place %d is outside its %d tokens of this step", i, j, lens[i]));
        std::vector<int> before(B), after(B);
        for (int i = 0; i < B; i++) {
            before[i] = (int)cache->length(slots[i]);
            after[i] = before[i] + lens[i];
            if (after[i] > model.max_positions)
                throw StepError(fmt("sequence %d: %d tokens after this step, the model has %d positions", i, after[i], model.max_positions));
        }
        cache->grow(slots, lens);                    // throws CacheFull before anything ran
        try {
            if (!is_prefill && use_graphs && graph_safe_) return decode_step(slots, tokens, want, before, after, greedy, chained);
            if (chained) throw StepError("a step that takes its ids from the device needs the captured decode path");
            return eager_step(slots, tokens, want, before, after, lens, is_prefill, greedy);
        } catch (...) {
            cache->shrink(slots, lens);              // the cache must not claim tokens whose keys were never written
            throw;
        }
    }

    // One token each for `slots`, the tokens being the greedy choice of an earlier step, still on the device (the host
    // may read them later): the next step of a generation loop is queued before the last one's tokens have arrived.
    bool can_chain() const { return use_graphs && graph_safe_; }
    StepResult step_chained(const std::vector<int>& slots, const DeviceIds& from) {
        std::vector<std::vector<int>> tokens(slots.size(), std::vector<int>{0});
        return step(slots, tokens, nullptr, true, &from);
    }

    // Chosen ids from the device to the caller's memory, through a pinned buffer; returns when they have arrived.
    void read_ids(const int* dev_ids, int n, int* out) {
        if (n <= 0) return;
        ids_host_.reserve((size_t)n);
        cuda_ok(cudaMemcpyAsync(ids_host_.host, dev_ids, (size_t)n * 4, cudaMemcpyDeviceToHost, ops.stream), "reading the chosen tokens");
        synchronize();
        memcpy(out, ids_host_.host, (size_t)n * 4);
    }

    // Error words of the kernels with bounded waits: "" when no wait ever ran out.  Synchronises and clears them.
    std::string kernel_errors() {
        synchronize();
        std::string out;
        auto& K = Kernels::get();
        for (auto& name : K.loaded()) {
            const KernelLib& l = K.lib(name);
            const char* sym = name == "gemm_tc" ? "tb_gemm_tc_error" : name == "attention_decode" ? "tb_attn_decode_error"
                              : name.rfind("attention_prefill_tc@", 0) == 0 ? "tb_attn_prefill_tc_error" : nullptr;
            if (!sym) continue;
            const int v = l.sym<int (*)()>(sym)();
            if (v) {
                out += (out.empty() ? "" : "; ") + name + fmt(": error word %d (a bounded wait ran out)", v);
                if (name == "attention_decode") cudaMemset(tickets_.p, 0, Ops::TICKET_SLOTS * 4);
            }
        }
        return out;
    }
    // Runs `fn` with scratch from `a`: first dry (every launch left out, allocations only counted), then, with the arena
    // grown to what that pass asked for, for real.
    template <typename F> auto sized_run(Arena& a, F fn) -> decltype(fn()) {
        Arena* keep = ops.arena;
        ops.arena = &a;
        try {
            a.dry = true;
            a.begin_step();
            fn();
            a.dry = false;
            if (!a.fits_peaks()) {
                synchronize();                       // earlier work may still use the old allocation
                a.grow_to_peaks();
            }
            a.begin_step();
            auto r = fn();
            ops.arena = keep;
            return r;
        } catch (...) {
            a.dry = false;
            ops.arena = keep;
            throw;
        }
    }
    int graphs_captured() const {
        int n = 0;
        for (auto& kv : decode_) n += kv.second->exec != nullptr;
        return n;
    }

private:
    struct DecodeShape {
        int B = 0, bucket = 0;
        int uneven = 0;
        int hits = 0;
        InputBuffer in;
        Arena arena;
        std::vector<size_t> table_off;
        std::vector<int> widths;
        size_t ints = 0, ids_off = 0, pos_off = 0, tseq_off = 0, start_off = 0, after_off = 0, slot_off = 0, src_off = 0;
        std::vector<int> table_slots;
        long long table_epoch = -1;
        cudaGraphExec_t exec = nullptr;
        Mat logits;
        int* greedy = nullptr;
        long long n_kernels = 0;
        bool sized = false;
    };

    bool classify(const std::vector<int>& slots, const std::vector<std::vector<int>>& tokens) {
        if (slots.empty()) throw StepError("a step needs at least one sequence");
        if (std::set<int>(slots.begin(), slots.end()).size() != slots.size()) throw StepError("a slot appears twice in one step");
        if (tokens.size() != slots.size()) throw StepError(fmt("%zu slots but %zu token lists", slots.size(), tokens.size()));
        bool all_zero = true, all_pos = true, all_one = true;
        for (size_t i = 0; i < slots.size(); i++) {
            const long long l = cache->length(slots[i]);
            if (tokens[i].empty()) throw StepError("every sequence of a step brings at least one token");
            all_zero &= l == 0; all_pos &= l > 0; all_one &= tokens[i].size() == 1;
        }
        if (all_zero) return true;
        if (all_pos && all_one) return false;
        throw StepError("the sequences of a step either all start (empty cache, whole prompts) or all go on by exactly one token");
    }
    static size_t align4(size_t n) { return (n + 3) & ~(size_t)3; }

    void fill_tables(int* dst, int width, int gi, const std::vector<int>& slots) {
        for (size_t i = 0; i < slots.size(); i++) {
            const auto& pg = cache->pages(slots[i], gi);
            for (size_t p = 0; p < pg.size() && (int)p < width; p++) dst[i * width + p] = pg[p];
        }
    }
    std::vector<CacheLine> lines_for(const std::vector<const int*>& tables, const std::vector<int>& widths) {
        std::vector<CacheLine> lines;
        for (size_t e = 0; e < model.schedule.size(); e++) {
            const int owner = model.schedule[e].cache_of < 0 ? (int)e : model.schedule[e].cache_of;
            CacheLine l = cache->line((int)e, owner);
            if (cache->has_line(owner)) {
                const int gi = cache->group_of(owner).first;
                l.page_table = tables[gi];
                l.pt_stride = widths[gi];
            }
            lines.push_back(l);
        }
        return lines;
    }

    StepResult eager_step(const std::vector<int>& slots, const std::vector<std::vector<int>>& tokens,
                          const std::vector<std::vector<int>>& want, const std::vector<int>& before, const std::vector<int>& after,
                          const std::vector<int>& lens, bool is_prefill, bool greedy) {
        const int B = (int)slots.size();
        int T = 0, n_want = 0, max_after = 0, max_len = 0;
        for (int i = 0; i < B; i++) { T += lens[i]; n_want += (int)want[i].size(); max_after = std::max(max_after, after[i]); max_len = std::max(max_len, lens[i]); }
        const size_t G = cache->groups().size();
        std::vector<int> widths(G);
        size_t ints = 0;
        const size_t ids_off = ints; ints += align4(T);
        const size_t pos_off = ints; ints += align4(T);
        const size_t tseq_off = ints; ints += align4(T);
        const size_t start_off = ints; ints += align4(B + 1);
        const size_t after_off = ints; ints += align4(B);
        const size_t slot_off = ints; ints += align4(B);
        const size_t want_off = ints; ints += align4(std::max(1, n_want));
        std::vector<size_t> table_off(G);
        for (size_t gi = 0; gi < G; gi++) { widths[gi] = cache->table_width((int)gi, max_after); table_off[gi] = ints; ints += align4((size_t)B * widths[gi]); }
        in_.reserve(ints);
        in_.wait();
        int* h = in_.host;
        memset(h, 0, ints * 4);
        bool all_rows = n_want == T;
        int t = 0, w = 0;
        for (int i = 0; i < B; i++) {
            h[start_off + i] = t;
            for (int j : want[i]) { h[want_off + w] = t + j; all_rows &= (t + j == w); w++; }
            for (int j = 0; j < lens[i]; j++, t++) { h[ids_off + t] = tokens[i][j]; h[pos_off + t] = before[i] + j; h[tseq_off + t] = i; }
            h[after_off + i] = after[i];
            h[slot_off + i] = slots[i];
        }
        h[start_off + B] = T;
        for (size_t gi = 0; gi < G; gi++) fill_tables(h + table_off[gi], widths[gi], (int)gi, slots);
        in_.upload(ints, ops.stream);
        h2d_bytes_last = (long long)ints * 4;

        StepCtx ctx;
        ctx.is_prefill = is_prefill; ctx.n_tokens = T; ctx.batch = B;
        ctx.positions = in_.d(pos_off); ctx.token_seq = in_.d(tseq_off); ctx.seq_start = in_.d(start_off);
        ctx.len_after = in_.d(after_off); ctx.slot_ids = in_.d(slot_off);
        ctx.slots = slots; ctx.seq_lens = lens; ctx.max_seq_len = max_len; ctx.max_len_after = max_after;
        ctx.len_bucket = len_bucket(max_after); ctx.uneven = is_prefill ? 0 : unevenness(after);
        std::vector<const int*> tables(G);
        for (size_t gi = 0; gi < G; gi++) tables[gi] = in_.d(table_off[gi]);
        std::vector<CacheLine> lines = lines_for(tables, widths);

        const int* want_rows = (n_want == 0 || !all_rows) ? in_.d(want_off) : nullptr;
        auto run = [&]() -> StepResult {
            StepCtx c = ctx;
            Mat logits = model.forward(ops, in_.d(ids_off), c, *cache, lines, want_rows, n_want);
            StepResult r;
            r.rows = n_want;
            if (n_want == 0) return r;
            if (greedy) r.ids = ops.argmax(logits);
            else r.logits = (const float*)logits.p;
            return r;
        };
        // a step of a shape not seen before first runs dry, to learn how much scratch it takes
        const auto shape = std::make_tuple(is_prefill, T, B, n_want, greedy);
        if (!sized_shapes_.count(shape)) {
            StepResult r = sized_run(arena_, run);
            if (sized_shapes_.size() < 4096) sized_shapes_.insert(shape);
            return r;
        }
        ops.arena = &arena_;
        arena_.begin_step();
        return run();
    }

    StepResult decode_step(const std::vector<int>& slots, const std::vector<std::vector<int>>& tokens,
                           const std::vector<std::vector<int>>& want, const std::vector<int>& before, const std::vector<int>& after,
                           bool greedy, const DeviceIds* chained = nullptr) {
        const int B = (int)slots.size();
        int max_after = 0;
        for (int a : after) max_after = std::max(max_after, a);
        const int bucket = len_bucket(max_after);
        const int uneven = unevenness(after);
        auto key = std::make_tuple(B, bucket, uneven);
        auto it = decode_.find(key);
        if (it == decode_.end()) it = decode_.emplace(key, make_shape(B, bucket, uneven)).first;
        DecodeShape& d = *it->second;
        // inputs
        d.in.wait();
        int* h = d.in.host;
        for (int i = 0; i < B; i++) {
            h[d.ids_off + i] = tokens[i][0];
            h[d.pos_off + i] = before[i];
            h[d.after_off + i] = after[i];
            h[d.slot_off + i] = slots[i];
        }
        // the page tables change only when the batch's slots change or any slot or page of the cache changes hands
        if (d.table_epoch != cache->epoch || d.table_slots != slots) {
            d.table_epoch = cache->epoch;
            d.table_slots = slots;
            for (size_t gi = 0; gi < d.widths.size(); gi++) fill_tables(h + d.table_off[gi], d.widths[gi], (int)gi, slots);
        }
        bool same_rows = false;
        if (chained) {
            if ((int)chained->src_rows.size() != B) throw StepError("a chained step needs one source row per sequence");
            same_rows = chained->n_src == B;
            for (int i = 0; i < B; i++) {
                if (chained->src_rows[i] < 0 || chained->src_rows[i] >= chained->n_src) throw StepError("a chained step's source row is out of range");
                same_rows &= chained->src_rows[i] == i;
                h[d.src_off + i] = chained->src_rows[i];
            }
        }
        d.in.upload(d.ints, ops.stream);
        h2d_bytes_last = (long long)d.ints * 4;
        if (chained) {
            // the ids come from the device, after the copy of the other inputs
            int* dst = (int*)d.in.dev.p + d.ids_off;
            if (same_rows) cuda_ok(cudaMemcpyAsync(dst, chained->ids, (size_t)B * 4, cudaMemcpyDeviceToDevice, ops.stream), "chaining ids");
            else ops.gather_rows_into(chained->ids, d.in.d(d.src_off), dst, B, 1, chained->n_src);
        }
        d.hits++;

        StepCtx ctx;
        ctx.is_prefill = false; ctx.n_tokens = B; ctx.batch = B;
        ctx.positions = d.in.d(d.pos_off); ctx.token_seq = d.in.d(d.tseq_off); ctx.seq_start = d.in.d(d.start_off);
        ctx.len_after = d.in.d(d.after_off); ctx.slot_ids = d.in.d(d.slot_off);
        ctx.slots = slots; ctx.seq_lens.assign(B, 1); ctx.max_seq_len = 1; ctx.max_len_after = max_after;
        ctx.len_bucket = bucket; ctx.uneven = uneven;
        std::vector<const int*> tables(d.widths.size());
        for (size_t gi = 0; gi < d.widths.size(); gi++) tables[gi] = d.in.d(d.table_off[gi]);
        std::vector<CacheLine> lines = lines_for(tables, d.widths);

        ops.arena = &d.arena;
        auto run = [&]() {
            d.arena.begin_step();
            StepCtx c = ctx;
            d.logits = model.forward(ops, d.in.d(d.ids_off), c, *cache, lines, nullptr, B);
            d.greedy = ops.argmax(d.logits);         // the greedy choice rides along
        };
        if (!d.sized) {
            d.arena.dry = true;
            run();
            d.arena.dry = false;
            if (!d.arena.fits_peaks()) d.arena.grow_to_peaks();
            d.sized = true;
        }
        if (!d.exec && d.hits >= 2) {
            // the first step of a shape ran eagerly (it also set up every kernel); the second is captured
            // (on the engine's own stream: the caller's may be the legacy default stream, which cannot capture)
            cudaGraph_t graph = nullptr;
            cudaStream_t run_stream = ops.stream;
            ops.stream = own_stream_;
            cudaError_t e = cudaStreamBeginCapture(own_stream_, cudaStreamCaptureModeThreadLocal);
            if (e != cudaSuccess) { ops.stream = run_stream; cuda_ok(e, "graph capture"); }
            try {
                run();
            } catch (...) {
                cudaStreamEndCapture(own_stream_, &graph);
                if (graph) cudaGraphDestroy(graph);
                ops.stream = run_stream;
                ops.arena = &arena_;
                throw;
            }
            ops.stream = run_stream;
            cuda_ok(cudaStreamEndCapture(own_stream_, &graph), "graph capture");
            cuda_ok(cudaGraphInstantiate(&d.exec, graph, 0), "graph instantiate");
            cudaGraphDestroy(graph);
        }
        if (d.exec) {
            cuda_ok(cudaGraphLaunch(d.exec, ops.stream), "graph launch");
            Kernels::get().launches += d.n_kernels;
        } else {
            const long long n0 = Kernels::get().launches;
            run();
            d.n_kernels = Kernels::get().launches - n0;
        }
        ops.arena = &arena_;
        StepResult r;
        std::vector<int> rows;
        for (int i = 0; i < B; i++)
            for (size_t k = 0; k < want[i].size(); k++) rows.push_back(i);
        r.rows = (int)rows.size();
        if (rows.empty()) return r;
        bool identity = (int)rows.size() == B;
        for (int i = 0; identity && i < B; i++) identity = rows[i] == i;
        if (identity) {
            if (greedy) r.ids = d.greedy;
            else r.logits = (const float*)d.logits.p;
            return r;
        }
        // a subset (or a repetition) of the rows: gathered outside the graph
        in_.reserve(rows.size());
        in_.wait();
        memcpy(in_.host, rows.data(), rows.size() * 4);
        in_.upload(rows.size(), ops.stream);
        return sized_run(arena_, [&]() {
            StepResult g;
            g.rows = (int)rows.size();
            Mat m = ops.gather_rows(d.logits, in_.d(0), (int)rows.size());
            if (greedy) g.ids = ops.argmax(m);
            else g.logits = (const float*)m.p;
            return g;
        });
    }

    std::unique_ptr<DecodeShape> make_shape(int B, int bucket, int uneven) {
        std::unique_ptr<DecodeShape> d(new DecodeShape);
        d->B = B; d->bucket = bucket; d->uneven = uneven;
        const long long cap = std::min<long long>(model.max_positions, cache->max_tokens());
        size_t ints = 0;
        d->ids_off = ints; ints += align4(B);
        d->pos_off = ints; ints += align4(B);
        d->tseq_off = ints; ints += align4(B);
        d->start_off = ints; ints += align4(B + 1);
        d->after_off = ints; ints += align4(B);
        d->slot_off = ints; ints += align4(B);
        d->src_off = ints; ints += align4(B);
        for (size_t gi = 0; gi < cache->groups().size(); gi++) {
            d->widths.push_back(cache->table_width((int)gi, cap));
            d->table_off.push_back(ints);
            ints += align4((size_t)B * d->widths.back());
        }
        d->ints = ints;
        d->in.reserve(ints);
        memset(d->in.host, 0, d->in.cap * 4);
        for (int i = 0; i < B; i++) { d->in.host[d->tseq_off + i] = i; d->in.host[d->start_off + i] = i; }
        d->in.host[d->start_off + B] = B;
        d->arena.reserve(1 << 16, 1 << 16);
        return d;
    }

    Arena arena_;
    InputBuffer in_, ids_host_;
    DeviceBuffer tickets_;
    cudaStream_t own_stream_ = nullptr;
    bool graph_safe_ = true;
    std::set<std::tuple<bool, int, int, int, bool>> sized_shapes_;
    std::map<std::tuple<int, int, int>, std::unique_ptr<DecodeShape>> decode_;
};

// ---- sampling options and the generation loop ------------------------------------------------------------------------
// Names and meanings as the reference's server has them (runtime/src/bin/serve.rs:1284-1292): temperature (<= 0: greedy),
// top_p, repetition_penalty (> 1 penalises the last 128 tokens), max_tokens; the seed is ours (the reference seeds from the
// wall clock, serve.rs:309-311).
struct SamplingParams {
    float temperature = 0.f, top_p = 0.95f, repetition_penalty = 1.f;
    int max_tokens = 256;
    unsigned long long seed = 0;
    bool greedy() const { return !(temperature > 0.f); }
    bool needs_sampler() const { return !greedy() || repetition_penalty > 1.f; }
};

constexpr int REPETITION_WINDOW = 128;

inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
// The draw u in [0, 1) for token `index` of request `request`: counter-based, so a request's samples do not depend
// on which batch it ran in.
inline float draw_uniform(uint64_t seed, uint64_t request, uint64_t index) {
    uint64_t x = mix64(seed);
    x = mix64(x ^ (request + 1));
    x = mix64(x ^ ((index + 1) * 0xD6E8FEB86659FD93ull));
    return (float)(x >> 40) / (float)(1 << 24);
}

// Cut requests, in order, into batches: at most max_batch sequences, and room in the cache for every sequence's
// prompt plus max_new tokens (counted in whole pages).
inline std::vector<std::vector<int>> plan_batches(const std::vector<int>& prompt_lens, int max_new, int max_batch, long long max_tokens,
                                                  int max_positions) {
    if (max_batch < 1) throw Error("max_batch must be at least 1");
    const int budget = pages_for(max_tokens);
    std::vector<std::vector<int>> batches;
    std::vector<int> cur;
    int used = 0;
    for (size_t i = 0; i < prompt_lens.size(); i++) {
        const int n = prompt_lens[i];
        if (n < 1) throw Error(fmt("request %zu: the prompt is empty", i));
        if (n > max_positions) throw Error(fmt("request %zu: a prompt of %d tokens exceeds the model's %d positions", i, n, max_positions));
        const int need = pages_for(std::min(n + max_new, max_positions));
        if (need > budget)
            throw Error(fmt("request %zu: %d prompt tokens plus %d new ones need %d cache tokens, the cache holds %d", i, n, max_new,
                            need * PAGE_ROWS, budget * PAGE_ROWS));
        if (!cur.empty() && ((int)cur.size() >= max_batch || used + need > budget)) { batches.push_back(cur); cur.clear(); used = 0; }
        cur.push_back((int)i);
        used += need;
    }
    if (!cur.empty()) batches.push_back(cur);
    return batches;
}

// Chosen ids on their way from the device to the host: the copy is queued at once, the host waits for it later.
struct IdsReader {
    int* host = nullptr;
    size_t cap = 0;
    cudaEvent_t done = nullptr;
    ~IdsReader() {
        if (host) cudaFreeHost(host);
        if (done) cudaEventDestroy(done);
    }
    void start(Engine& eng, const int* dev_ids, int n) {
        if ((size_t)n > cap) {
            if (host) cudaFreeHost(host);
            cap = std::max<size_t>(256, (size_t)n * 2);
            cuda_ok(cudaMallocHost((void**)&host, cap * 4), "pinned ids");
        }
        if (!done) cuda_ok(cudaEventCreateWithFlags(&done, cudaEventDisableTiming), "event");
        cuda_ok(cudaMemcpyAsync(host, dev_ids, (size_t)n * 4, cudaMemcpyDeviceToHost, eng.ops.stream), "reading the chosen tokens");
        cuda_ok(cudaEventRecord(done, eng.ops.stream), "event");
    }
    const int* wait() {
        cuda_ok(cudaEventSynchronize(done), "waiting for the chosen tokens");
        return host;
    }
};

typedef int (*OnToken)(int request, int token, void* user);        // a non-zero return ends the generation

// Generate up to params.max_tokens new ids for every prompt.  A sequence ends at a stop id (which is not emitted,
// runtime/src/bin/serve.rs:347-350), after max_tokens new tokens, or at the model's context limit; its slot and pages go
// back at once and the batch shrinks.  The next batch starts when the last sequence of this one has ended.
inline std::vector<std::vector<int>> generate(Engine& eng, const std::vector<std::vector<int>>& prompts, const SamplingParams& p,
                                              const std::vector<int>* stop_ids, int max_batch, OnToken on_token, void* user) {
    if (!(p.top_p > 0.f)) throw Error("top_p must be positive");
    if (!(p.repetition_penalty > 0.f)) throw Error("repetition_penalty must be positive");
    if (p.max_tokens < 0) throw Error("max_tokens must not be negative");
    std::vector<std::vector<int>> outputs(prompts.size());
    if (p.max_tokens == 0 || prompts.empty()) return outputs;
    std::set<int> stops(stop_ids ? stop_ids->begin() : eng.model.stop_ids.begin(), stop_ids ? stop_ids->end() : eng.model.stop_ids.end());
    std::vector<int> lens;
    for (auto& q : prompts) lens.push_back((int)q.size());
    const bool greedy = !p.needs_sampler();
    const int max_pos = eng.model.max_positions;
    struct Seq { int request, slot, length; std::deque<int> recent; int count = 0; std::vector<int> out; int row = 0; bool queued = false; };
    DeviceBuffer fbuf, rbuf;
    Arena sample_arena;
    sample_arena.reserve(1 << 16, 256);
    std::vector<float> fhost;
    std::vector<int> rhost, chosen;
    bool stop_all = false;
    for (auto& batch : plan_batches(lens, p.max_tokens, std::min(max_batch, eng.cache->max_slots()), eng.cache->max_tokens(), max_pos)) {
        std::vector<int> slots = eng.start((int)batch.size());
        std::vector<Seq> live;
        for (size_t i = 0; i < batch.size(); i++) {
            Seq s;
            s.request = batch[i]; s.slot = slots[i]; s.length = lens[batch[i]];
            const auto& pr = prompts[batch[i]];
            for (size_t k = pr.size() > (size_t)REPETITION_WINDOW ? pr.size() - REPETITION_WINDOW : 0; k < pr.size(); k++) s.recent.push_back(pr[k]);
            live.push_back(std::move(s));
        }
        try {
            std::vector<std::vector<int>> toks;
            for (auto& s : live) toks.push_back(prompts[s.request]);
            StepResult r = eng.step(slots, toks, nullptr, greedy);
            int steps = 0;
            if (greedy && eng.can_chain()) {
                // Greedy decoding, pipelined: the next step is queued with its ids taken on the device (the choice that
                // the step before it made) before the host has read those ids.  The host reads them one step behind,
                // emits them and decides who goes on.  What it cannot know ahead is a stop id: a sequence that turns
                // out to have stopped was stepped once too often, which costs one row of one step and nothing else
                // (its slot and pages go back; that row's result is never read).
                IdsReader readers[2];
                int cur = 0;
                for (size_t i = 0; i < live.size(); i++) live[i].row = (int)i;
                readers[cur].start(eng, r.ids, r.rows);
                while (!live.empty()) {
                    // who goes on unless the pending token turns out to be a stop id
                    std::vector<int> next_slots;
                    DeviceIds from;
                    from.ids = r.ids; from.n_src = r.rows;
                    for (auto& s : live) {
                        const bool known_last = (int)s.out.size() + 1 >= p.max_tokens || s.length + 1 > max_pos - 1;
                        s.queued = !known_last && !stop_all;
                        if (s.queued) { next_slots.push_back(s.slot); from.src_rows.push_back(s.row); }
                    }
                    StepResult r2;
                    if (!next_slots.empty()) {
                        r2 = eng.step_chained(next_slots, from);
                        readers[cur ^ 1].start(eng, r2.ids, r2.rows);
                    }
                    const int* ids = readers[cur].wait();
                    std::vector<Seq> next;
                    int next_row = 0;
                    for (auto& s : live) {
                        const int tok = ids[s.row];
                        const bool is_stop = stops.count(tok) != 0;
                        if (!is_stop) {
                            s.out.push_back(tok);
                            if (on_token && on_token(s.request, tok, user)) stop_all = true;
                        }
                        const int row2 = s.queued ? next_row++ : -1;
                        if (s.queued && !is_stop && !stop_all) {
                            s.row = row2;
                            s.length++;
                            next.push_back(std::move(s));
                        } else {
                            outputs[s.request] = s.out;
                            eng.release({s.slot});
                        }
                    }
                    live = std::move(next);
                    r = r2;
                    cur ^= 1;
                    steps++;
                    if (live.empty() || steps % 64 == 0) {
                        const std::string err = eng.kernel_errors();
                        if (!err.empty()) throw Error("a kernel gave up waiting and its results are not valid: " + err);
                    }
                }
            }
            while (!live.empty()) {
                const int rows = (int)live.size();
                chosen.resize(rows);
                if (greedy) {
                    eng.read_ids(r.ids, rows, chosen.data());
                } else {
                    // per row: temperature, top_p, penalty, draw; and the recent tokens if there is a penalty
                    fhost.resize(4 * rows);
                    for (int i = 0; i < rows; i++) {
                        fhost[i] = p.temperature; fhost[rows + i] = p.top_p; fhost[2 * rows + i] = p.repetition_penalty;
                        fhost[3 * rows + i] = draw_uniform(p.seed, (uint64_t)live[i].request, (uint64_t)live[i].count);
                    }
                    if (fbuf.bytes < fhost.size() * 4) fbuf.alloc(fhost.size() * 4 * 2);
                    cuda_ok(cudaMemcpyAsync(fbuf.p, fhost.data(), fhost.size() * 4, cudaMemcpyHostToDevice, eng.ops.stream), "sampling inputs");
                    const int* recent = nullptr;
                    if (p.repetition_penalty > 1.f) {
                        rhost.assign((size_t)rows * REPETITION_WINDOW, -1);
                        for (int i = 0; i < rows; i++) std::copy(live[i].recent.begin(), live[i].recent.end(), rhost.begin() + (size_t)i * REPETITION_WINDOW);
                        if (rbuf.bytes < rhost.size() * 4) rbuf.alloc(rhost.size() * 4 * 2);
                        cuda_ok(cudaMemcpyAsync(rbuf.p, rhost.data(), rhost.size() * 4, cudaMemcpyHostToDevice, eng.ops.stream), "sampling inputs");
                        recent = (const int*)rbuf.p;
                    }
                    const float* f = (const float*)fbuf.p;
                    Mat logits((void*)r.logits, F32, rows, eng.model.vocab);
                    // the sampling kernels' scratch lies outside the step's arena, which still holds the logits
                    int* ids = eng.sized_run(sample_arena, [&]() {
                        return eng.ops.sample(logits, f, f + rows, f + 2 * rows, f + 3 * rows, recent, REPETITION_WINDOW, p.top_p < 1.f);
                    });
                    eng.read_ids(ids, rows, chosen.data());
                }
                std::vector<Seq> next;
                for (int i = 0; i < rows; i++) {
                    Seq& s = live[i];
                    const int tok = chosen[i];
                    s.recent.push_back(tok);
                    if ((int)s.recent.size() > REPETITION_WINDOW) s.recent.pop_front();
                    s.count++;
                    // why the sequence ends once `tok` has been chosen, if it does
                    const bool is_stop = stops.count(tok) != 0;
                    const bool last = !is_stop && ((int)s.out.size() + 1 >= p.max_tokens || s.length + 1 > max_pos - 1);
                    if (!is_stop) {
                        s.out.push_back(tok);
                        if (on_token && on_token(s.request, tok, user)) stop_all = true;
                    }
                    if (is_stop || last || stop_all) {
                        outputs[s.request] = s.out;
                        eng.release({s.slot});
                    } else next.push_back(std::move(s));
                }
                live = std::move(next);
                if (!live.empty()) {
                    std::vector<int> sl;
                    std::vector<std::vector<int>> one;
                    for (auto& s : live) { sl.push_back(s.slot); one.push_back({s.out.back()}); }
                    r = eng.step(sl, one, nullptr, greedy);
                    for (auto& s : live) s.length++;
                }
                steps++;
                if (live.empty() || steps % 64 == 0) {
                    // the chosen tokens were just read on the host: a kernel whose bounded wait ran out must not pass
                    // its garbage on as tokens
                    const std::string err = eng.kernel_errors();
                    if (!err.empty()) throw Error("a kernel gave up waiting and its results are not valid: " + err);
                }
            }
        } catch (...) {
            for (auto& s : live)
                if (eng.cache->slot_held(s.slot)) eng.cache->release(s.slot);
            throw;
        }
        if (stop_all) break;
    }
    return outputs;
}

}  // namespace tb

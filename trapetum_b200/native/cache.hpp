// The cache: keys and values per layer call, pages per sequence, state per slot.
//
// Every schedule entry that owns a cache declares what it needs (keys and values per token, or a state of fixed
// size).  Entries with the same key/value geometry and the same window form a group; a group has one allocation
// [lines, pages, kv_heads, PAGE_ROWS, head_dim] for keys, one for values, and one page pool, because all its
// lines grow in step: page p of a sequence is page p in every line of the group.  A group with window W is a
// ring of ceil(W / PAGE_ROWS) * PAGE_ROWS rows per sequence (row = position mod ring).  A sequence takes a slot
// when it starts and pages as it grows; release gives all of it back and the next sequence reuses the numbers
// (lowest free number first; freeing what is not held is an error).  The reference has one flat cache per layer
// for its single sequence (runtime/src/lib.rs:4475) and nothing to hand out.
#pragma once
#include <queue>
#include <set>
#include <tuple>

#include "ops.hpp"

namespace tb {

struct CacheFull : Error {
    using Error::Error;
};

class Pool {
public:
    Pool(int capacity, std::string what) : capacity_(capacity), what_(std::move(what)), held_(capacity, false) {
        for (int i = 0; i < capacity; i++) free_.push(i);
    }
    int capacity() const { return capacity_; }
    int free_count() const { return (int)free_.size(); }
    int held_count() const { return capacity_ - (int)free_.size(); }
    std::vector<int> take(int n) {
        if (n > (int)free_.size())
            throw CacheFull(fmt("%s pool: %d asked, %zu of %d free", what_.c_str(), n, free_.size(), capacity_));
        std::vector<int> out;
        for (int i = 0; i < n; i++) { out.push_back(free_.top()); free_.pop(); held_[out.back()] = true; }
        return out;
    }
    void give_back(const std::vector<int>& ids) {
        std::set<int> seen;
        for (int i : ids) {
            if (i < 0 || i >= capacity_ || !held_[i])
                throw Error(fmt("%s pool: %d is not held (freed twice, or never taken)", what_.c_str(), i));
            if (!seen.insert(i).second) throw Error(fmt("%s pool: %d is given back twice in one call", what_.c_str(), i));
        }
        for (int i : ids) { held_[i] = false; free_.push(i); }
    }
    bool is_held(int i) const { return i >= 0 && i < capacity_ && held_[i]; }

private:
    int capacity_;
    std::string what_;
    std::priority_queue<int, std::vector<int>, std::greater<int>> free_;
    std::vector<bool> held_;
};

struct CacheNeed {
    enum Kind { NONE, KV, STATE } kind = NONE;
    int n_kv_heads = 0, head_dim = 0, window = 0;      // KV: window 0 keeps every token
    size_t state_bytes = 0;                            // STATE: bytes per sequence, zeroed when a sequence starts
};

inline int pages_for(long long tokens) { return (int)((tokens + PAGE_ROWS - 1) / PAGE_ROWS); }

struct KVGroup {
    int n_kv_heads, head_dim, window, ring_rows;
    std::vector<int> entries;
    std::unique_ptr<Pool> pool;
    DeviceBuffer k, v;                   // [lines, pages, kv_heads, PAGE_ROWS, head_dim]
    size_t line_bytes = 0;
    int n_pages = 0;
    int rows_held(long long len) const { return (int)(ring_rows ? std::min<long long>(len, ring_rows) : len); }
};

class Cache {
public:
    // `needs`: owning schedule entry -> need; `readers`: owning entry -> has readers.  `max_tokens`: the most tokens
    // that live sequences hold at any time, each sequence's count rounded up to PAGE_ROWS.  `device` false: only the
    // bookkeeping (no storage), for use without a GPU.
    Cache(const std::map<int, CacheNeed>& needs, const std::set<int>& shared, long long max_tokens, DType dt, int max_slots,
          bool device = true)
        : dt_(dt), shared_(shared) {
        if (max_tokens <= 0) throw Error(fmt("cache: max_tokens must be positive, got %lld", max_tokens));
        n_pages_ = pages_for(max_tokens);
        max_tokens_ = (long long)n_pages_ * PAGE_ROWS;
        max_slots_ = std::min(n_pages_, max_slots > 0 ? max_slots : 1024);
        slots_.reset(new Pool(max_slots_, "slot"));
        std::map<std::tuple<int, int, int>, std::vector<int>> by_key;
        for (auto& kv : needs) {
            if (kv.second.kind == CacheNeed::KV) by_key[{kv.second.n_kv_heads, kv.second.head_dim, kv.second.window}].push_back(kv.first);
            else if (kv.second.kind == CacheNeed::STATE) {
                State st;
                st.bytes = kv.second.state_bytes;
                if (device) {
                    st.buf.alloc(st.bytes * max_slots_);
                    cuda_ok(cudaMemset(st.buf.p, 0, st.bytes * max_slots_), "zeroing the state area");
                }
                states_[kv.first] = std::move(st);
            }
        }
        for (auto& kv : by_key) {
            KVGroup g;
            std::tie(g.n_kv_heads, g.head_dim, g.window) = kv.first;
            g.entries = kv.second;
            g.ring_rows = g.window ? pages_for(g.window) * PAGE_ROWS : 0;
            // a ring never holds more than ring_rows per sequence, so its pool can be smaller
            g.n_pages = g.ring_rows ? std::min(n_pages_, max_slots_ * (g.ring_rows / PAGE_ROWS)) : n_pages_;
            g.pool.reset(new Pool(g.n_pages, "page"));
            g.line_bytes = (size_t)g.n_pages * g.n_kv_heads * PAGE_ROWS * g.head_dim * dtype_size(dt);
            if (device) { g.k.alloc(g.line_bytes * g.entries.size()); g.v.alloc(g.line_bytes * g.entries.size()); }
            for (size_t i = 0; i < g.entries.size(); i++) entry_group_[g.entries[i]] = {(int)groups_.size(), (int)i};
            groups_.push_back(std::move(g));
        }
    }

    long long epoch = 0;                 // counts every change of who holds which slot or page
    int max_slots() const { return max_slots_; }
    long long max_tokens() const { return max_tokens_; }
    std::vector<KVGroup>& groups() { return groups_; }
    bool slot_held(int s) const { return len_.count(s) != 0; }

    int claim(cudaStream_t stream = nullptr) {
        const int slot = slots_->take(1)[0];
        epoch++;
        len_[slot] = 0;
        pages_[slot].assign(groups_.size(), {});
        for (auto& kv : states_)
            if (kv.second.buf.p)
                cuda_ok(cudaMemsetAsync((char*)kv.second.buf.p + kv.second.bytes * slot, 0, kv.second.bytes, stream), "zeroing a state");
        return slot;
    }
    long long length(int slot) const { held(slot); return len_.at(slot); }
    const std::vector<int>& pages(int slot, int group) const { held(slot); return pages_.at(slot).at(group); }

    // Make room for growth[i] more tokens of slots[i]: all of it or nothing.
    void grow(const std::vector<int>& slots, const std::vector<int>& growth) {
        struct Want { int slot, group, add; };
        std::vector<Want> want;
        std::vector<int> per_group(groups_.size(), 0);
        for (size_t i = 0; i < slots.size(); i++) {
            held(slots[i]);
            if (growth[i] < 0) throw Error(fmt("slot %d: cannot grow by %d", slots[i], growth[i]));
            const long long new_len = len_[slots[i]] + growth[i];
            for (size_t gi = 0; gi < groups_.size(); gi++) {
                const int add = pages_for(groups_[gi].rows_held(new_len)) - (int)pages_[slots[i]][gi].size();
                if (add > 0) { want.push_back({slots[i], (int)gi, add}); per_group[gi] += add; }
            }
        }
        for (size_t gi = 0; gi < groups_.size(); gi++)
            if (per_group[gi] > groups_[gi].pool->free_count()) {
                long long held_tokens = 0;
                for (auto& kv : len_) held_tokens += kv.second;
                throw CacheFull(fmt("the cache is full: this step needs %d more pages of %d tokens, %d of %d are free (%zu live "
                                    "sequences hold %lld tokens; the cache was sized for %lld)", per_group[gi], PAGE_ROWS,
                                    groups_[gi].pool->free_count(), groups_[gi].pool->capacity(), len_.size(), held_tokens, max_tokens_));
            }
        for (auto& w : want) {
            auto got = groups_[w.group].pool->take(w.add);
            auto& pg = pages_[w.slot][w.group];
            pg.insert(pg.end(), got.begin(), got.end());
        }
        if (!want.empty()) epoch++;
        for (size_t i = 0; i < slots.size(); i++) len_[slots[i]] += growth[i];
    }
    // Undo a grow whose step did not run.
    void shrink(const std::vector<int>& slots, const std::vector<int>& growth) {
        for (size_t i = 0; i < slots.size(); i++) {
            held(slots[i]);
            if (growth[i] < 0 || growth[i] > len_[slots[i]]) throw Error(fmt("slot %d: cannot shrink by %d", slots[i], growth[i]));
        }
        for (size_t i = 0; i < slots.size(); i++) {
            len_[slots[i]] -= growth[i];
            for (size_t gi = 0; gi < groups_.size(); gi++) {
                auto& pg = pages_[slots[i]][gi];
                const size_t keep = (size_t)pages_for(groups_[gi].rows_held(len_[slots[i]]));
                if (pg.size() > keep) {
                    groups_[gi].pool->give_back(std::vector<int>(pg.begin() + keep, pg.end()));
                    pg.resize(keep);
                }
            }
        }
        epoch++;
    }
    void release(int slot) {
        held(slot);
        for (size_t gi = 0; gi < groups_.size(); gi++) groups_[gi].pool->give_back(pages_[slot][gi]);
        pages_.erase(slot);
        len_.erase(slot);
        slots_->give_back({slot});
        epoch++;
    }
    std::vector<int> live_slots() const {
        std::vector<int> v;
        for (auto& kv : len_) v.push_back(kv.first);
        return v;
    }
    // Bookkeeping invariants: no page lost, none held twice.
    void check() const {
        for (size_t gi = 0; gi < groups_.size(); gi++) {
            std::set<int> seen;
            size_t n = 0;
            for (auto& kv : pages_)
                for (int p : kv.second[gi]) { seen.insert(p); n++; }
            if (seen.size() != n) throw Error(fmt("group %zu: a page belongs to two sequences", gi));
            if ((int)n != groups_[gi].pool->held_count())
                throw Error(fmt("group %zu: %d pages are taken, sequences hold %zu", gi, groups_[gi].pool->held_count(), n));
        }
        if ((int)len_.size() != slots_->held_count()) throw Error("slots: the pool and the sequences disagree");
    }
    int table_width(int group, long long max_len) const { return std::max(1, pages_for(groups_[group].rows_held(max_len))); }

    bool has_line(int owner) const { return entry_group_.count(owner) != 0; }
    std::pair<int, int> group_of(int owner) const { return entry_group_.at(owner); }
    // The view of one schedule entry; the page table of the running batch is filled in by the engine.
    CacheLine line(int entry, int owner) {
        CacheLine l;
        auto it = entry_group_.find(owner);
        if (it != entry_group_.end()) {
            KVGroup& g = groups_[it->second.first];
            l.k = (char*)g.k.p + g.line_bytes * it->second.second;
            l.v = (char*)g.v.p + g.line_bytes * it->second.second;
            l.ring_rows = g.ring_rows; l.n_kv_heads = g.n_kv_heads; l.head_dim = g.head_dim; l.dt = dt_;
        }
        auto st = states_.find(owner);
        if (st != states_.end()) { l.state = st->second.buf.p; l.state_bytes = st->second.bytes; }
        l.entry = owner; l.owner = entry == owner; l.shared = shared_.count(owner) != 0;
        return l;
    }

private:
    struct State { DeviceBuffer buf; size_t bytes = 0; };
    void held(int slot) const {
        if (!len_.count(slot)) throw Error(fmt("slot %d is not held by any sequence", slot));
    }
    DType dt_;
    int n_pages_ = 0, max_slots_ = 0;
    long long max_tokens_ = 0;
    std::unique_ptr<Pool> slots_;
    std::vector<KVGroup> groups_;
    std::map<int, std::pair<int, int>> entry_group_;
    std::map<int, State> states_;
    std::set<int> shared_;
    std::map<int, long long> len_;
    std::map<int, std::vector<std::vector<int>>> pages_;
};

}  // namespace tb

// The operations of a step as the host sees them: each checks what its kernel relies on, picks the kernel
// (tensor cores or 32-bit FMA, which attention kernel, how many pieces) and launches it on the step's stream
// with scratch taken from the step's arena.  No CPU path stands behind any of them.
#pragma once
#include "kernels.hpp"

namespace tb {

struct CacheLine {                       // what a mixer call sees of the cache (one line of a group)
    void* k = nullptr;                   // [pages, kv_heads, PAGE_ROWS, head_dim]
    void* v = nullptr;
    const int* page_table = nullptr;     // device int32 [batch, pt_stride]
    int pt_stride = 0;
    int ring_rows = 0;
    int n_kv_heads = 0, head_dim = 0;
    DType dt = BF16;
    int entry = 0;                       // the owning schedule entry
    bool owner = true;                   // this call writes the line
    bool shared = false;                 // some later call reads this line
    void* state = nullptr;               // per-slot state of the entry, if it has one: [max_slots, state_bytes]
    size_t state_bytes = 0;
};

struct StepCtx {                         // what the parts may know about the running step
    bool is_prefill = false;
    int n_tokens = 0, batch = 0;
    const int* positions = nullptr;      // device int32 [tokens]
    const int* token_seq = nullptr;      // [tokens]
    const int* seq_start = nullptr;      // [batch + 1]
    const int* len_after = nullptr;      // [batch]
    const int* slot_ids = nullptr;       // [batch]
    std::vector<int> slots, seq_lens;    // host copies
    int max_seq_len = 0, max_len_after = 0, len_bucket = 0;
    int uneven = 0;                  // decode: how much the contexts differ in length, 0..3
    std::map<int, std::pair<Mat, Mat>> step_kv;      // prefill: entry -> (k, v) of this step
};

enum Activation { GELU_TANH = 0, SILU = 1 };

inline int activation_code(const std::string& name) {
    if (name == "gelu_tanh") return GELU_TANH;
    if (name == "silu") return SILU;
    throw Error("unknown activation '" + name + "' (known: gelu_tanh, silu)");
}

class Ops {
public:
    Arena* arena = nullptr;
    cudaStream_t stream = nullptr;
    int sms = 148;
    int* tickets = nullptr;              // zeroed counters of the decode attention's fold
    static constexpr int TICKET_SLOTS = 1 << 16;
    bool dry() const { return arena->dry; }

    // ---- embedding, rows -------------------------------------------------------------------------------
    Mat embed(const int* ids, const Mat& table, float scale, int n) {
        Mat out = arena->mat(F32, n, table.cols);
        if (dry()) return out;
        auto& l = K().lib("embed");
        static auto f = l.sym<int (*)(const int*, const void*, int, float*, int, int, int, float, cudaStream_t)>("tb_embed");
        launched(l, f(ids, table.p, table.dt, (float*)out.p, n, (int)table.cols, (int)table.rows, scale, stream), "embed");
        return out;
    }
    Mat gather_rows(const Mat& x, const int* rows, int n) {
        need(x.dt == F32 && x.contiguous(), "gather_rows: x must be contiguous float32");
        Mat out = arena->mat(F32, n, x.cols);
        if (dry()) return out;
        auto& l = K().lib("embed");
        static auto f = l.sym<int (*)(const float*, const int*, float*, int, int, int, cudaStream_t)>("tb_gather_rows");
        launched(l, f((const float*)x.p, rows, (float*)out.p, n, (int)x.cols, (int)x.rows, stream), "gather_rows");
        return out;
    }

    // out[i] = in[rows[i]] for rows of `width` 32-bit words, into memory of the caller's
    void gather_rows_into(const void* in, const int* rows, void* out, int n, int width, int n_rows) {
        if (dry()) return;
        auto& l = K().lib("embed");
        static auto f = l.sym<int (*)(const float*, const int*, float*, int, int, int, cudaStream_t)>("tb_gather_rows");
        launched(l, f((const float*)in, rows, (float*)out, n, width, n_rows, stream), "gather_rows");
    }

    // ---- norms -----------------------------------------------------------------------------------------
    Mat rmsnorm(const Mat& x, const Mat& w, float eps, float offset, DType out_dt) {
        need(x.contiguous() && w.cols == x.cols, "rmsnorm: x and w do not fit");
        Mat out = arena->mat(out_dt, x.rows, x.cols);
        if (dry()) return out;
        auto& l = K().lib("norm");
        static auto f = l.sym<int (*)(const void*, int, const void*, int, void*, int, int, int, float, float, cudaStream_t)>("tb_rmsnorm");
        launched(l, f(x.p, x.dt, w.p, w.dt, out.p, out_dt, (int)x.rows, (int)x.cols, eps, offset, stream), "rmsnorm");
        return out;
    }
    // h += norm_a(a) in place; with wb also returns norm_b(h).  `a`: partial sums (added in split order on the way).
    Mat add_rmsnorm(const Mat& h, const Partials& a, const Mat& wa, float eps_a, float off_a, const Mat* wb, float eps_b,
                    float off_b, DType out_dt) {
        need(h.dt == F32 && h.contiguous() && a.rows == h.rows && a.cols == h.cols, "add_rmsnorm: shapes do not fit");
        need(!wb || wb->dt == wa.dt, "add_rmsnorm: both norm weights must have one dtype");
        Mat out;
        if (wb) out = arena->mat(out_dt, h.rows, h.cols);
        if (dry()) return out;
        auto& l = K().lib("norm");
        static auto f = l.sym<int (*)(float*, const void*, int, int, long long, const void*, float, float, const void*, float,
                                      float, int, void*, int, int, int, cudaStream_t)>("tb_add_rmsnorm");
        launched(l, f((float*)h.p, a.p, F32, a.splits, a.split_stride, wa.p, eps_a, off_a, wb ? wb->p : nullptr, eps_b, off_b,
                      wa.dt, out.p, wb ? (int)out_dt : 0, (int)h.rows, (int)h.cols, stream), "add_rmsnorm");
        return out;
    }
    void residual_add(const Mat& h, const Partials& a) {
        Mat s = sum_partials(a);
        if (dry()) return;
        auto& l = K().lib("norm");
        static auto f = l.sym<int (*)(float*, const void*, int, long long, cudaStream_t)>("tb_residual_add");
        launched(l, f((float*)h.p, s.p, F32, (long long)h.rows * h.cols, stream), "residual_add");
    }
    Mat sum_partials(const Partials& a) {
        if (a.splits == 1) return a.first();
        Mat out = arena->mat(F32, a.rows, a.cols);
        if (dry()) return out;
        need(a.split_stride == a.rows * a.cols, "sum_partials: partial sums must be contiguous");
        auto& l = K().lib("gemm_tc");
        static auto f = l.sym<int (*)(const float*, float*, int, int, int, cudaStream_t)>("tb_sum_partials");
        launched(l, f(a.p, (float*)out.p, (int)a.rows, (int)a.cols, a.splits, stream), "sum_partials");
        return out;
    }

    // ---- elementwise -----------------------------------------------------------------------------------
    Mat gated_act(const Mat& gu, int act, DType out_dt) {
        need(gu.contiguous() && gu.cols % 2 == 0, "gated_act: input must be contiguous [rows, 2*intermediate]");
        Mat out = arena->mat(out_dt, gu.rows, gu.cols / 2);
        if (dry()) return out;
        auto& l = K().lib("activation");
        static auto f = l.sym<int (*)(const void*, int, void*, int, int, int, int, cudaStream_t)>("tb_gated_act");
        launched(l, f(gu.p, gu.dt, out.p, out_dt, (int)gu.rows, (int)(gu.cols / 2), act, stream), "gated_act");
        return out;
    }
    void add_bias(const Mat& x, const Mat& bias) {
        need(bias.cols == x.cols, "add_bias: bias does not fit the rows");
        if (dry()) return;
        auto& l = K().lib("activation");
        static auto f = l.sym<int (*)(void*, int, long long, const void*, int, int, int, cudaStream_t)>("tb_add_bias");
        launched(l, f(x.p, x.dt, x.ld, bias.p, bias.dt, (int)x.rows, (int)x.cols, stream), "add_bias");
    }

    // ---- matrix products: y[T, N] = x[T, K] @ W[N, K]^T ------------------------------------------------
    static bool gemm_tc_takes(const Mat& a, const Mat& w) {
        if (a.dt != BF16 || w.dt != BF16 || a.cols != w.cols) return false;
        return a.cols % 8 == 0 && a.ld % 8 == 0 && w.ld % 8 == 0 && ((uintptr_t)a.p % 16) == 0 && ((uintptr_t)w.p % 16) == 0;
    }
    Mat gemm_simt(const Mat& a, const Mat& w, DType out_dt, float cap) {
        need(a.cols == w.cols, "gemm: inner sizes differ");
        Mat out = arena->mat(out_dt, a.rows, w.rows);
        if (dry()) return out;
        auto& l = K().lib("gemm_simt");
        static auto f = l.sym<int (*)(const void*, int, const void*, int, void*, int, int, int, int, long long, long long,
                                      long long, float, cudaStream_t)>("tb_gemm_simt");
        launched(l, f(a.p, a.dt, w.p, w.dt, out.p, out_dt, (int)a.rows, (int)w.rows, (int)a.cols, a.ld, w.ld, out.ld, cap, stream),
                 "gemm_simt");
        return out;
    }
    int gemm_tc_splits(const Mat& a, const Mat& w) {
        auto& l = K().lib("gemm_tc");
        static auto pick = l.sym<int (*)(int, int, int, int)>("tb_gemm_tc_splits");
        static auto eff = l.sym<int (*)(int, int)>("tb_gemm_tc_effective_splits");
        return eff((int)a.cols, pick((int)a.rows, (int)w.rows, (int)a.cols, sms));
    }
    typedef int (*gemm_tc_fn)(const void*, const void*, void*, int, int, int, int, long long, long long, long long, float, int,
                              float*, int, int, cudaStream_t);
    gemm_tc_fn gemm_tc_entry(const KernelLib& l) {
        static auto f = l.sym<gemm_tc_fn>("tb_gemm_tc");
        return f;
    }
    Mat gemm_tc(const Mat& a, const Mat& w, DType out_dt, float cap) {
        const int splits = gemm_tc_splits(a, w);
        Mat out = arena->mat(out_dt, a.rows, w.rows);
        float* scratch = splits > 1 ? (float*)arena->alloc((size_t)splits * a.rows * w.rows * 4) : nullptr;
        if (dry()) return out;
        auto& l = K().lib("gemm_tc");
        launched(l, gemm_tc_entry(l)(a.p, w.p, out.p, out_dt, (int)a.rows, (int)w.rows, (int)a.cols, a.ld, w.ld, out.ld, cap,
                                     splits, scratch, 1, -1, stream), "gemm_tc", splits > 1 ? 2 : 1);
        return out;
    }
    Partials gemm_tc_partials(const Mat& a, const Mat& w) {
        const int splits = gemm_tc_splits(a, w);
        Partials part;
        part.splits = splits; part.rows = a.rows; part.cols = w.rows; part.split_stride = a.rows * w.rows;
        part.p = (float*)arena->alloc((size_t)splits * a.rows * w.rows * 4);
        if (dry()) return part;
        auto& l = K().lib("gemm_tc");
        if (splits == 1)
            launched(l, gemm_tc_entry(l)(a.p, w.p, part.p, 0, (int)a.rows, (int)w.rows, (int)a.cols, a.ld, w.ld, w.rows, 0.f, 1,
                                         nullptr, 1, -1, stream), "gemm_tc");
        else
            launched(l, gemm_tc_entry(l)(a.p, w.p, nullptr, 0, (int)a.rows, (int)w.rows, (int)a.cols, a.ld, w.ld, w.rows, 0.f,
                                         splits, part.p, 0, -1, stream), "gemm_tc");
        return part;
    }
    // w holds gate and up rows interleaved in blocks of 16; the result is bfloat16 [M, N/2] = act(gate) * up
    Mat gemm_tc_gated(const Mat& a, const Mat& w, int act) {
        need(w.rows % 32 == 0, "gemm_tc: the gated epilogue needs a multiple of 32 weight rows");
        Mat out = arena->mat(BF16, a.rows, w.rows / 2);
        if (dry()) return out;
        auto& l = K().lib("gemm_tc");
        launched(l, gemm_tc_entry(l)(a.p, w.p, out.p, 1, (int)a.rows, (int)w.rows, (int)a.cols, a.ld, w.ld, out.ld, 0.f, 1,
                                     nullptr, 1, act, stream), "gemm_tc");
        return out;
    }
    // the one place that picks a GEMM kernel
    Mat linear(const Mat& x, const Mat& w, DType out_dt, float cap = 0.f) {
        if (gemm_tc_takes(x, w)) return gemm_tc(x, w, out_dt, cap);
        return gemm_simt(x, w, out_dt, cap);
    }
    Partials linear_partials(const Mat& x, const Mat& w) {
        if (gemm_tc_takes(x, w)) return gemm_tc_partials(x, w);
        Mat y = gemm_simt(x, w, F32, 0.f);
        Partials p;
        p.p = (float*)y.p; p.splits = 1; p.rows = y.rows; p.cols = y.cols; p.split_stride = y.rows * y.cols;
        return p;
    }

    // ---- rotation and cache write ------------------------------------------------------------------------
    void rope_kv(const Mat& qkv, int n_heads, int n_kv_heads, int head_dim, int rotary_dim, const float* inv_freq,
                 const StepCtx& ctx, const CacheLine* store, const Partials* partial) {
        need(qkv.cols == (int64_t)(n_heads + 2 * n_kv_heads) * head_dim, "rope_kv: qkv width does not fit the head counts");
        if (dry()) return;
        RopeKvArgs a;
        memset(&a, 0, sizeof a);
        a.qkv = qkv.p; a.row_stride = qkv.ld;
        a.q_off = 0; a.k_off = n_heads * head_dim; a.v_off = (n_heads + n_kv_heads) * head_dim;
        a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.rotary_dim = rotary_dim;
        a.inv_freq = inv_freq;
        a.positions = ctx.positions; a.token_seq = ctx.token_seq; a.len_after = ctx.len_after;
        if (store) {
            a.k_pool = store->k; a.v_pool = store->v; a.page_table = store->page_table; a.pt_stride = store->pt_stride;
            a.ring_rows = store->ring_rows;
        }
        a.page_rows = PAGE_ROWS;
        if (partial) {
            a.partial = partial->p; a.n_splits = partial->splits; a.split_stride = partial->split_stride;
            a.partial_row_stride = partial->cols;
        }
        auto& l = K().lib("rope_kv");
        static auto f = l.sym<int (*)(const RopeKvArgs*, int, int, cudaStream_t)>("tb_rope_kv");
        launched(l, f(&a, qkv.dt, (int)qkv.rows, stream), "rope_kv");
    }

    // ---- attention -----------------------------------------------------------------------------------------
    static bool attn_prefill_tc_takes(DType dt, int hd) { return dt == BF16 && (hd == 64 || hd == 128 || hd == 256); }
    static bool attn_prefill_mma_takes(DType dt, int hd) { return dt == BF16 && hd % 16 == 0 && hd >= 16 && hd <= 256; }
    Mat attn_prefill(const Mat& q, const Mat& k, const Mat& v, const StepCtx& ctx, int n_heads, int n_kv_heads, int hd,
                     float scale, float cap, int window) {
        need(k.ld == v.ld && k.dt == q.dt && v.dt == q.dt, "attention: k and v must share row stride and dtype with q");
        Mat out = arena->mat(q.dt, q.rows, (int64_t)n_heads * hd);
        if (dry()) return out;
        if (attn_prefill_tc_takes(q.dt, hd)) {
            auto& l = K().lib(fmt("attention_prefill_tc@TB_HD=%d", hd));
            auto f = l.sym<int (*)(const void*, const void*, const void*, long long, long long, const int*, void*, int, int, int,
                                   int, int, int, float, float, int, cudaStream_t)>("tb_attn_prefill_tc");
            launched(l, f(q.p, k.p, v.p, q.ld, k.ld, ctx.seq_start, out.p, (int)q.rows, ctx.batch, ctx.max_seq_len, n_heads,
                          n_kv_heads, hd, scale, cap, window, stream), "attn_prefill_tc", 2);
        } else if (attn_prefill_mma_takes(q.dt, hd)) {
            auto& l = K().lib(fmt("attention_prefill@TB_HD=%d", hd));
            auto f = l.sym<int (*)(const void*, const void*, const void*, long long, long long, const int*, void*, int, int, int,
                                   int, int, float, float, int, cudaStream_t)>("tb_attn_prefill_mma");
            launched(l, f(q.p, k.p, v.p, q.ld, k.ld, ctx.seq_start, out.p, ctx.batch, ctx.max_seq_len, n_heads, n_kv_heads, hd,
                          scale, cap, window, stream), "attn_prefill_mma");
        } else {
            auto& l = K().lib("attention_simt");
            static auto f = l.sym<int (*)(const void*, const void*, const void*, long long, long long, const int*, const int*,
                                          void*, int, int, int, int, int, float, float, int, cudaStream_t)>("tb_attn_prefill_simt");
            launched(l, f(q.p, k.p, v.p, q.ld, k.ld, ctx.seq_start, ctx.token_seq, out.p, q.dt, (int)q.rows, n_heads, n_kv_heads,
                          hd, scale, cap, window, stream), "attn_prefill_simt");
        }
        return out;
    }

    static bool attn_decode_takes(DType dt, int n_heads, int n_kv, int hd) {
        if (dt != BF16 || n_kv <= 0 || n_heads % n_kv) return false;
        const int g = n_heads / n_kv;
        return ((hd == 64 || hd == 128 || hd == 256) && g >= 1 && g <= 8) || (hd == 32 && (g == 1 || g == 2 || g == 4 || g == 8));
    }
    static bool attn_decode_rotates(DType dt, int n_heads, int n_kv, int hd) { return attn_decode_takes(dt, n_heads, n_kv, hd) && hd >= 64; }
    static bool attn_decode_stream_takes(DType dt, int n_heads, int n_kv, int hd, int batch) {
        return attn_decode_takes(dt, n_heads, n_kv, hd) && hd >= 64 && batch <= 1024 && batch * n_kv <= TICKET_SLOTS;
    }
    // Whether decode attention deals its pages out as one stream (see csrc/ops.py: decode_partition_is_stream).
    static bool decode_partition_is_stream(int batch, int n_kv, int pages, int splits, int uneven, int sms) {
        const int per = (pages + splits - 1) / splits;
        return uneven * per >= 4 * 10 || batch * n_kv * splits > 2 * sms;
    }
    // 0: chosen per launch; 1: the split partition, 2: the stream partition (tests, comparisons)
    static int& decode_partition_override() {
        static int mode = 0;
        return mode;
    }

    // In how many pieces decode attention cuts a sequence's pages (see csrc/ops.py: choose_decode_splits).
    static int choose_decode_splits(int batch, int n_kv, int pages, int sms) {
        const int items = std::max(1, batch * n_kv);
        int best = 1;
        double best_eff = 0.0;
        for (int s = 1; s <= std::max(1, pages / 4); s++) {
            if (s > 64) break;
            const int ctas = items * s;
            double eff = (double)ctas / ((double)((ctas + sms - 1) / sms) * sms);
            const int per = (pages + s - 1) / s;
            eff *= per / (per + 4.0);
            if (eff > best_eff + 1e-9) { best = s; best_eff = eff; }
        }
        return best;
    }
    // One query per sequence against the paged cache.  `q`: the rotated queries [B, n_heads*hd] with the new token's
    // k, v already stored; or, with `part`, the q/k/v product's partial sums, which the kernel adds, rotates
    // (inv_freq, rotary_dim) and appends to the cache itself.
    Mat attn_decode(const Mat* q, const Partials* part, const float* inv_freq, int rotary_dim, const CacheLine& line,
                    const StepCtx& ctx, int n_heads, int n_kv, int hd, float scale, float cap, int window) {
        const int B = q ? (int)q->rows : (int)part->rows;
        const DType dt = q ? q->dt : BF16;
        const int rows = line.ring_rows ? std::min(ctx.len_bucket, line.ring_rows) : ctx.len_bucket;
        const int pages = std::max(1, (rows + PAGE_ROWS - 1) / PAGE_ROWS);
        const int splits = choose_decode_splits(B, n_kv, pages, sms);
        Mat out = arena->mat(dt, B, (int64_t)n_heads * hd);
        DecodeArgs a;
        memset(&a, 0, sizeof a);
        if (q) { a.q = q->p; a.q_stride = q->ld; }
        a.k_pool = line.k; a.v_pool = line.v; a.page_table = line.page_table; a.pt_stride = line.pt_stride;
        a.len_after = ctx.len_after; a.out = out.p;
        a.n_heads = n_heads; a.n_kv_heads = n_kv; a.hd = hd; a.page_rows = PAGE_ROWS;
        a.ring_rows = line.ring_rows; a.window = window; a.scale = scale; a.cap = cap;
        if (part) {
            need(part->cols == (int64_t)(n_heads + 2 * n_kv) * hd, "attention: the q/k/v partial sums have the wrong width");
            a.qkv_part = part->p; a.qkv_splits = part->splits; a.qkv_split_stride = part->split_stride;
            a.qkv_row_stride = part->cols; a.inv_freq = inv_freq; a.rotary_dim = inv_freq ? rotary_dim : 0;
        }
        bool one_stream = decode_partition_is_stream(B, n_kv, pages, splits, ctx.uneven, sms);
        if (decode_partition_override()) one_stream = decode_partition_override() == 2;
        if (one_stream && attn_decode_stream_takes(dt, n_heads, n_kv, hd, B)) {
            auto& l = K().lib("attention_decode");
            static auto nf = l.sym<long long (*)(int, int, int, int)>("tb_attn_decode_stream_scratch_floats");
            static auto f = l.sym<int (*)(const DecodeArgs*, int, int, int, cudaStream_t)>("tb_attn_decode_stream");
            static auto nc = l.sym<int (*)(int, int)>("tb_attn_decode_stream_ctas");
            const int n_ctas = nc(sms, hd);
            a.partial = (float*)arena->alloc((size_t)nf(n_ctas, n_heads, n_kv, hd) * 4);
            a.n_splits = 0; a.tickets = tickets;
            if (dry()) return out;
            launched(l, f(&a, dt, B, n_ctas, stream), "attn_decode_stream");
            return out;
        }
        if (attn_decode_takes(dt, n_heads, n_kv, hd)) {
            const bool mma = hd >= 64;
            need(mma || !part, "attention: only the tensor-core decode kernel rotates by itself");
            a.n_splits = splits;
            if (splits > 1) a.partial = (float*)arena->alloc((size_t)B * n_heads * splits * (hd + 2) * 4);
            const bool fused_fold = mma && splits > 1 && B * n_kv <= TICKET_SLOTS;
            a.tickets = fused_fold ? tickets : nullptr;
            if (dry()) return out;
            auto& l = K().lib("attention_decode");
            static auto f_mma = l.sym<int (*)(const DecodeArgs*, int, int, cudaStream_t)>("tb_attn_decode");
            static auto f_lanes = l.sym<int (*)(const DecodeArgs*, int, int, cudaStream_t)>("tb_attn_decode_lanes");
            launched(l, (mma ? f_mma : f_lanes)(&a, dt, B, stream), "attn_decode", (splits > 1 && !fused_fold) ? 2 : 1);
            return out;
        }
        need(!part, "attention: this shape's decode kernel does not rotate by itself");
        a.n_splits = splits;
        if (splits > 1) a.partial = (float*)arena->alloc((size_t)B * n_heads * splits * (hd + 2) * 4);
        if (dry()) return out;
        auto& l = K().lib("attention_simt");
        static auto f = l.sym<int (*)(const DecodeArgs*, int, int, cudaStream_t)>("tb_attn_decode_simt");
        launched(l, f(&a, dt, B, stream), "attn_decode_simt");
        return out;
    }

    // ---- choosing tokens -------------------------------------------------------------------------------------
    int* argmax(const Mat& logits) {
        need(logits.dt == F32, "argmax: logits must be float32");
        auto& l = K().lib("sampling");
        static auto nb = l.sym<long long (*)(int, int)>("tb_argmax_scratch_bytes");
        static auto f = l.sym<int (*)(const float*, long long, int, int, int*, void*, cudaStream_t)>("tb_argmax");
        void* scratch = arena->alloc((size_t)std::max<long long>(8, nb((int)logits.rows, (int)logits.cols)));
        int* out = (int*)arena->alloc((size_t)logits.rows * 4);
        if (dry()) return out;
        launched(l, f((const float*)logits.p, logits.ld, (int)logits.rows, (int)logits.cols, out, scratch, stream), "argmax", 2);
        return out;
    }
    static constexpr int WIDE_SAMPLING_FROM = 16384;
    // per row: repetition penalty over `recent` (changes the logits in place), then argmax if the row's temperature
    // is <= 0, else a nucleus draw with the row's `draw` in [0, 1)
    int* sample(const Mat& logits, const float* temperature, const float* top_p, const float* penalty, const float* draw,
                const int* recent, int n_recent, bool nucleus) {
        auto& l = K().lib("sampling");
        static auto nb = l.sym<long long (*)(int, int)>("tb_sample_wide_scratch_bytes");
        static auto fw = l.sym<int (*)(const SampleArgs*, int, void*, int, cudaStream_t)>("tb_sample_wide");
        static auto fs = l.sym<int (*)(const SampleArgs*, int, cudaStream_t)>("tb_sample");
        int* out = (int*)arena->alloc((size_t)logits.rows * 4);
        SampleArgs a;
        memset(&a, 0, sizeof a);
        a.logits = (float*)logits.p; a.row_stride = logits.ld; a.vocab = (int)logits.cols;
        a.temperature = temperature; a.top_p = top_p; a.penalty = penalty; a.draw = draw;
        a.recent = recent; a.n_recent = recent ? n_recent : 0; a.out = out;
        if (logits.cols >= WIDE_SAMPLING_FROM) {
            void* scratch = arena->alloc((size_t)nb((int)logits.rows, (int)logits.cols));
            if (dry()) return out;
            launched(l, fw(&a, (int)logits.rows, scratch, nucleus ? 1 : 0, stream), "sample", nucleus ? 10 : 4);
            return out;
        }
        if (dry()) return out;
        launched(l, fs(&a, (int)logits.rows, stream), "sample");
        return out;
    }

    // ---- weights made on the device ------------------------------------------------------------------------
    void random_normal(void* out, DType dt, long long n, unsigned k0, unsigned k1, float std) {
        auto& l = K().lib("random_init");
        static auto f = l.sym<int (*)(void*, int, long long, unsigned, unsigned, float, cudaStream_t)>("tb_random_normal");
        launched(l, f(out, dt, n, k0, k1, std, stream), "random_normal");
    }

    static void need(bool ok, const char* what) {
        if (!ok) throw Error(what);
    }

private:
    static Kernels& K() { return Kernels::get(); }
    void launched(const KernelLib& l, int status, const char* what, int kernels = 1) {
        Kernels::check(l, status, what);
        K().launches += kernels;
    }
};

}  // namespace tb

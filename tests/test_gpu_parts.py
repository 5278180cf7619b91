"""The parts of a layer, each alone against the plain implementation; and the generality of the
arrangement: a schedule that names a layer twice and shares a cache, and a toy mixer with a state of
its own that is registered, built and stepped without touching the library."""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_gemma2 as plain
from conftest import TINY_A, TINY_B, TINY_C, TOL, bf16_budget, make_prompts, rel_l2, sharpen

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def _whole(y):
    """A part may return [splits, tokens, hidden] partial sums; their sum is the result."""
    return y.sum(0) if y.dim() == 3 else y


def _rt(dt):
    from trapetum_b200.parts import Runtime
    return Runtime(dt, torch.device("cuda:0"))


def _ctx(lens_before, new, slots=None):
    from trapetum_b200.engine.step import StepContext
    B, T = len(new), sum(new)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    after = [b + n for b, n in zip(lens_before, new)]
    return StepContext(is_prefill=all(b == 0 for b in lens_before), n_tokens=T, batch=B,
                       positions=dev([p for b, n in zip(lens_before, new) for p in range(b, b + n)]),
                       token_seq=dev([i for i, n in enumerate(new) for _ in range(n)]), seq_start=dev(starts),
                       len_after=dev(after), slot_ids=dev(slots or list(range(B))), slots=slots or list(range(B)),
                       seq_lens=list(new), max_seq_len=max(new), max_len_after=max(after), len_bucket=256)


@pytest.mark.parametrize("dt", DTYPES)
def test_norm_part_and_stream(dt):
    from trapetum_b200.config import PartSpec
    from trapetum_b200.parts import ResidualStream, build_part
    H = 200
    mk = lambda n, eps, uo: build_part("norm", PartSpec("rmsnorm", {"size": H, "eps": eps, "unit_offset": uo, "weight": n}),
                                       "p.", _rt(dt))
    n1, n2, n3 = mk("a", 1e-6, True), mk("b", 1e-5, True), mk("c", 1e-6, False)
    assert list(n1.tensor_specs()) == ["p.a"] and n1.tensor_specs()["p.a"].shape == (H,)
    w = {f"p.{k}": (torch.randn(H, device="cuda") * 0.3).to(dt) for k in "abc"}
    for n in (n1, n2, n3):
        n.bind(w)
    h0 = torch.randn(7, H, device="cuda")
    a = (torch.randn(7, H, device="cuda") * 4).to(dt)
    b = (torch.randn(7, H, device="cuda") * 4).to(dt)
    st = ResidualStream(h0.clone())
    x1 = st.normed(n1, dt)
    st.add_normed(a, n2)
    x2 = st.normed(n3, dt)                      # the addition and the next norm run as one kernel
    st.add(b)
    hf = st.value()
    pw = {k: v.float().cpu() for k, v in w.items()}
    ph = h0.cpu()
    assert rel_l2(x1, plain.rmsnorm(ph, pw["p.a"], 1e-6)) < (1e-6 if dt == torch.float32 else 5e-3)
    ph = ph + plain.rmsnorm(a.float().cpu(), pw["p.b"], 1e-5)
    want3 = ph * torch.rsqrt((ph * ph).mean(-1, keepdim=True) + 1e-6) * pw["p.c"]
    assert rel_l2(x2, want3) < (1e-6 if dt == torch.float32 else 5e-3)
    assert rel_l2(hf, ph + b.float().cpu()) < 1e-6


@pytest.mark.parametrize("dt", DTYPES)
def test_feed_forward_part(dt):
    from trapetum_b200.config import PartSpec
    from trapetum_b200.parts import build_part
    H, I = 136, 392
    ff = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "gelu_tanh",
                                                           "gate": "g", "up": "u", "down": "d"}), "L.", _rt(dt))
    specs = ff.tensor_specs()
    assert specs["L.g"].shape == (I, H) and specs["L.d"].shape == (H, I)
    w = {"L.g": torch.randn(I, H) * 0.1, "L.u": torch.randn(I, H) * 0.1, "L.d": torch.randn(H, I) * 0.1}
    w = {k: v.bfloat16() for k, v in w.items()}
    ff.bind({k: v.to("cuda", dt) for k, v in w.items()})
    x = torch.randn(150, H).bfloat16()
    got = ff.forward(x.to("cuda", dt), None)
    assert got.dtype == torch.float32
    got = _whole(got)
    want = plain.feed_forward(x.float(), w["L.g"].float(), w["L.u"].float(), w["L.d"].float())
    assert rel_l2(got, want) < (1e-5 if dt == torch.float32 else 1e-2)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C])
def test_attention_part_prefill_then_decode(dt, cfg):
    """The attention mixer with its rope and its cache line, outside any model: a first step of two
    unequal sequences, then single tokens, against whole-sequence attention."""
    from trapetum_b200.cache import Cache
    from trapetum_b200.config import load_config
    from trapetum_b200.parts import build_part
    _, spec = load_config(cfg)
    layer = spec.layers[0]                                       # a sliding layer
    att = build_part("mixer", layer.mixer, layer.prefix, _rt(dt))
    H = cfg["hidden_size"]
    w = {n: (torch.randn(s.shape) * 0.15).bfloat16() for n, s in att.tensor_specs().items()}
    att.bind({k: v.to("cuda", dt) for k, v in w.items()})
    cache = Cache({0: att.cache_need()}, {}, 64 * 8, dt, "cuda")
    lens = [cfg["sliding_window"] + 5, 3]
    extra = 6
    xs = [torch.randn(n + extra, H).bfloat16() for n in lens]
    pw = {k: v.float() for k, v in w.items()}
    pcfg = dict(cfg)
    want = [plain.attention_block(x.float(), pw, layer.prefix, pcfg, cfg["sliding_window"])[0] for x in xs]
    slots = [cache.claim(), cache.claim()]
    cache.grow({s: n for s, n in zip(slots, lens)})

    def table(max_len):
        width = cache.table_width(0, max_len)
        t = torch.zeros(2, width, dtype=torch.int32)
        for i, s in enumerate(slots):
            pg = cache.pages(s, 0)
            t[i, :len(pg)] = torch.tensor(pg, dtype=torch.int32)
        cache.groups[0].table = t.cuda()
    table(max(lens))
    ctx = _ctx([0, 0], lens)
    x = torch.cat([xs[0][:lens[0]], xs[1][:lens[1]]]).to("cuda", dt)
    got = _whole(att.forward(x, ctx, cache.view(0, 0)))
    t = 1e-5 if dt == torch.float32 else 1.5e-2
    assert rel_l2(got[:lens[0]], want[0][:lens[0]]) < t and rel_l2(got[lens[0]:], want[1][:lens[1]]) < t
    for step in range(extra):
        before = [n + step for n in lens]
        cache.grow({s: 1 for s in slots})
        table(max(before) + 1)
        ctx = _ctx(before, [1, 1])
        x = torch.stack([xs[0][before[0]], xs[1][before[1]]]).to("cuda", dt)
        got = _whole(att.forward(x, ctx, cache.view(0, 0)))
        assert rel_l2(got[0], want[0][before[0]]) < t and rel_l2(got[1], want[1][before[1]]) < t


# ---------------------------------------------------------------------------
# A schedule that names a layer twice and lets a call read another call's cache
# ---------------------------------------------------------------------------
LOOPED = [(0, None), (1, None), (0, None), (1, 1)]


def _register_looped():
    from trapetum_b200.config import Gemma2Config, ModelSpec, ScheduleEntry, register_architecture
    from trapetum_b200.models.gemma2 import gemma2_spec

    def spec(cfg):
        s = gemma2_spec(cfg)
        return ModelSpec(**{**s.__dict__, "architecture": "TestLoopedGemma2",
                            "schedule": tuple(ScheduleEntry(l, c) for l, c in LOOPED)})
    register_architecture("TestLoopedGemma2", Gemma2Config, spec)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_repeats_a_layer_and_shares_a_cache(tmp_path, dtype):
    import trapetum_b200 as tb
    _register_looped()
    cfg = dict(TINY_A, architectures=["TestLoopedGemma2"])
    d = str(tmp_path / "looped")
    tb.write_random_model(d, cfg, 3, 0.05, 0.2)
    sharpen(d, 3.0)
    pc, pw = plain.load_folder(d)
    model = tb.load_model(d, dtype)
    eng = tb.Engine(model, 64 * 8)
    assert sum(g.k.shape[0] for g in eng.cache.groups) == 3        # entries 0, 1, 2 own lines; entry 3 reads entry 1's
    prompts = make_prompts(256, [30, 12], seed=8)
    truth = [plain.forward(pc, pw, p, schedule=LOOPED) for p in prompts]
    tol = TOL[dtype] if dtype == "float32" else bf16_budget(pc, pw, prompts, LOOPED)
    s = eng.start(2)
    cut = [18, 5]
    first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut])
    assert max(rel_l2(first[i], truth[0][i]) for i in range(18)) <= tol
    assert max(rel_l2(first[18 + i], truth[1][i]) for i in range(5)) <= tol
    for t in range(7):
        out = eng.step(s, [[prompts[0][18 + t]], [prompts[1][5 + t]]])
        assert rel_l2(out[0], truth[0][18 + t]) <= tol and rel_l2(out[1], truth[1][5 + t]) <= tol
    eng.release(s)


# ---------------------------------------------------------------------------
# A toy mixer with a state of its own, defined here
# ---------------------------------------------------------------------------
def _register_toy():
    from trapetum_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from trapetum_b200.config.base import _get
    from trapetum_b200.parts import Mixer, StateNeed, register_part
    from trapetum_b200.weights import TensorSpec

    class RunningMean(Mixer):
        """y_t = W * mean(x_0..x_t): its state is the running sum and the count, kept per sequence in
        the cache's state area.  Plain torch on the device: a toy, not a product kernel."""

        def __init__(self, params, prefix, rt):
            super().__init__(params, prefix, rt)
            self.h = params["hidden_size"]

        def tensor_specs(self):
            return {self._name("weight"): TensorSpec((self.h, self.h))}

        def bind(self, tensors):
            self.w = tensors[self._name("weight")].float()

        def cache_need(self):
            return StateNeed((self.h + 1,))

        def forward(self, x, ctx, state):
            x = x.float()
            out = torch.empty_like(x)
            start = 0
            for slot, n in zip(ctx.slots, ctx.seq_lens):
                st = state.data[slot]
                cs = torch.cumsum(x[start:start + n], 0) + st[:self.h]
                cnt = st[self.h] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[start:start + n] = cs / cnt[:, None]
                st[:self.h] = cs[-1]
                st[self.h] = cnt[-1]
                start += n
            return out @ self.w.T

    register_part("mixer", "test_running_mean", RunningMean)

    @dataclass(frozen=True)
    class ToyConfig:
        layers: int
        hidden: int
        inter: int
        vocab: int
        eps: float

        @classmethod
        def from_dict(cls, d):
            return cls(_get(d, "toy_layers", int), _get(d, "toy_hidden", int), _get(d, "toy_inter", int),
                       _get(d, "toy_vocab", int), _get(d, "toy_eps", float))

    def spec(c):
        norm = lambda n: PartSpec("rmsnorm", {"size": c.hidden, "eps": c.eps, "unit_offset": False, "weight": n})
        layers = tuple(LayerSpec(
            block=PartSpec("pre_norm", {"pre_mixer_norm": norm("n1.weight"), "pre_ffn_norm": norm("n2.weight")}),
            mixer=PartSpec("test_running_mean", {"hidden_size": c.hidden, "weight": "mix.weight"}),
            feed_forward=PartSpec("gated_mlp", {"hidden_size": c.hidden, "intermediate_size": c.inter, "activation": "silu",
                                                "gate": "g.weight", "up": "u.weight", "down": "d.weight"}),
            prefix=f"blocks.{i}.") for i in range(c.layers))
        return ModelSpec(architecture="TestToyLM", hidden_size=c.hidden, vocab_size=c.vocab,
                         embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.hidden, "scale": 1.0,
                                                          "weight": "emb.weight"}),
                         layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(c.layers)),
                         final_norm=norm("out_norm.weight"),
                         head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.hidden, "softcap": None,
                                                       "weight": "head.weight", "tied_to": None}),
                         max_positions=512)
    register_architecture("TestToyLM", ToyConfig, spec)


def _toy_plain(cfg, w, ids):
    """The toy model, whole sequence, plain torch on the CPU."""
    H, eps = cfg["toy_hidden"], cfg["toy_eps"]
    norm = lambda x, g: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * g
    h = w["emb.weight"][torch.tensor(ids)]
    for i in range(cfg["toy_layers"]):
        p = f"blocks.{i}."
        x = norm(h, w[p + "n1.weight"])
        mean = torch.cumsum(x, 0) / torch.arange(1, len(ids) + 1)[:, None]
        h = h + mean @ w[p + "mix.weight"].T
        x = norm(h, w[p + "n2.weight"])
        g = x @ w[p + "g.weight"].T
        h = h + ((g * torch.sigmoid(g)) * (x @ w[p + "u.weight"].T)) @ w[p + "d.weight"].T
    return norm(h, w["out_norm.weight"]) @ w["head.weight"].T


def test_a_toy_mixer_with_its_own_state_is_registered_built_and_stepped(tmp_path):
    import trapetum_b200 as tb
    _register_toy()
    cfg = {"architectures": ["TestToyLM"], "toy_layers": 2, "toy_hidden": 40, "toy_inter": 56, "toy_vocab": 90,
           "toy_eps": 1e-5}
    d = str(tmp_path / "toy")
    tb.write_random_model(d, cfg, 9, 0.2, 0.3)
    pw = plain.load_folder(d)[1]
    for k in pw:
        if "n1" in k or "n2" in k or "out_norm" in k:
            pw[k] = pw[k]                                          # plain (not 1+w) norms, as the spec says
    model = tb.load_model(d, "float32")
    eng = tb.Engine(model, 64 * 4, max_slots=4)
    assert eng.cache.groups == [] and sorted(eng.cache.states) == [0, 1]       # no keys or values: state only
    prompts = make_prompts(90, [21, 8, 13], seed=1)
    truth = [_toy_plain(cfg, pw, p) for p in prompts]
    for round_ in range(2):                                        # the second round reuses slots: state must restart
        s = eng.start(3)
        cut = [10, 8 - 3, 1]
        first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut])
        o = 0
        for r in range(3):
            assert max(rel_l2(first[o + i], truth[r][i]) for i in range(cut[r])) < 1e-5
            o += cut[r]
        live = list(range(3))
        t = 0
        while live:
            for r in [r for r in live if cut[r] + t >= len(prompts[r])]:
                eng.release([s[r]]); live.remove(r)
            if not live:
                break
            out = eng.step([s[r] for r in live], [[prompts[r][cut[r] + t]] for r in live])
            for i, r in enumerate(live):
                assert rel_l2(out[i], truth[r][cut[r] + t]) < 1e-5
            t += 1
    out = tb.generate(eng, [prompts[0][:4]], max_tokens=5, stop_ids=[])
    ids = list(prompts[0][:4])
    for tok in out[0]:
        assert tok == int(_toy_plain(cfg, pw, ids)[-1].argmax())
        ids.append(tok)


# ---------------------------------------------------------------------------
# A toy feed-forward with routing and a toy position encoding, defined here, around the library's attention
# ---------------------------------------------------------------------------
def _register_routed():
    from trapetum_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from trapetum_b200.config.base import _get
    from trapetum_b200.csrc import ops
    from trapetum_b200.parts import FeedForward, PositionEncoding, build_part, register_part
    from trapetum_b200.weights import TensorSpec

    class Damped(PositionEncoding):
        """q_t *= 1 + rise * t and k_j *= cos(swing * j): not a rotation, so it answers no rotary table and the
        attention part has to call it.  Plain torch on the device, then the library's cache write."""

        def __init__(self, params, prefix, rt):
            super().__init__(params, prefix, rt)
            self.head_dim, self.rise, self.swing = int(params["head_dim"]), float(params["rise"]), float(params["swing"])

        def kernel_files(self):
            return ("rope_kv",)

        def rotate_and_store(self, qkv, n_heads, n_kv_heads, ctx, line, store, partial=None):
            if partial is not None:
                qkv.copy_(partial.sum(0))
            pos = ctx.positions.float()[:, None]
            qw, kw = n_heads * self.head_dim, n_kv_heads * self.head_dim
            qkv[:, :qw] = (qkv[:, :qw].float() * (1.0 + self.rise * pos)).to(qkv.dtype)
            if kw:
                qkv[:, qw:qw + kw] = (qkv[:, qw:qw + kw].float() * torch.cos(self.swing * pos)).to(qkv.dtype)
            if store:
                ops.rope_kv(qkv, n_heads, n_kv_heads, self.head_dim, 0, None, ctx.positions, ctx.token_seq,
                            ctx.len_after, line.k, line.v, line.page_table, line.ring_rows)

    class Routed(FeedForward):
        """Each token goes to the expert with the largest router logit (32-bit), weighted by that logit's
        softmax probability; the experts are the library's gated feed-forwards.  All experts run on all
        tokens and a mask keeps the chosen one: a toy, with no launch that depends on host values."""

        def __init__(self, params, prefix, rt):
            super().__init__(params, prefix, rt)
            self.h, self.n = int(params["hidden_size"]), int(params["experts"])
            self.experts = [build_part("feed_forward", PartSpec("gated_mlp", {
                "hidden_size": self.h, "intermediate_size": int(params["intermediate_size"]), "activation": "silu",
                "gate": "g.weight", "up": "u.weight", "down": "d.weight"}), f"{prefix}experts.{e}.", rt)
                for e in range(self.n)]

        def tensor_specs(self):
            specs = {self._name("router"): TensorSpec((self.n, self.h))}
            for e in self.experts:
                specs.update(e.tensor_specs())
            return specs

        def bind(self, tensors):
            self.router = tensors[self._name("router")].float()
            for e in self.experts:
                e.bind(tensors)

        def kernel_files(self):
            return tuple(k for e in self.experts for k in e.kernel_files())

        def forward(self, x, ctx):
            p = torch.softmax(x.float() @ self.router.T, -1)                    # router in 32-bit
            top = p.argmax(-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e, part in enumerate(self.experts):
                y = _whole(part.forward(x, ctx)).float()
                out += y * (p[:, e] * (top == e))[:, None]
            return out

    register_part("position", "test_damped", Damped)
    register_part("feed_forward", "test_routed", Routed)

    @dataclass(frozen=True)
    class RoutedConfig:
        layers: int; hidden: int; heads: int; kv_heads: int; head_dim: int; inter: int; experts: int; vocab: int; eps: float

        @classmethod
        def from_dict(cls, d):
            g = lambda k, t=int: _get(d, "r_" + k, t)
            return cls(g("layers"), g("hidden"), g("heads"), g("kv_heads"), g("head_dim"), g("inter"), g("experts"),
                       g("vocab"), g("eps", float))

    def spec(c):
        norm = lambda n: PartSpec("rmsnorm", {"size": c.hidden, "eps": c.eps, "unit_offset": False, "weight": n})
        layers = tuple(LayerSpec(
            block=PartSpec("pre_norm", {"pre_mixer_norm": norm("n1.weight"), "pre_ffn_norm": norm("n2.weight")}),
            mixer=PartSpec("attention", {"hidden_size": c.hidden, "num_heads": c.heads, "num_kv_heads": c.kv_heads,
                                         "head_dim": c.head_dim, "scale": c.head_dim ** -0.5, "softcap": None,
                                         "window": None, "q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight",
                                         "position": PartSpec("test_damped", {"head_dim": c.head_dim, "rise": 0.01,
                                                                              "swing": 0.3})}),
            feed_forward=PartSpec("test_routed", {"hidden_size": c.hidden, "intermediate_size": c.inter,
                                                  "experts": c.experts, "router": "router.weight"}),
            prefix=f"blocks.{i}.") for i in range(c.layers))
        return ModelSpec(architecture="TestRoutedLM", hidden_size=c.hidden, vocab_size=c.vocab,
                         embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.hidden, "scale": 1.0,
                                                          "weight": "emb.weight"}),
                         layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(c.layers)),
                         final_norm=norm("out_norm.weight"),
                         head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.hidden, "softcap": None,
                                                       "weight": "head.weight", "tied_to": None}),
                         max_positions=512)
    register_architecture("TestRoutedLM", RoutedConfig, spec)


def _routed_plain(cfg, w, ids):
    """The routed toy model, whole sequence, plain torch on the CPU in 64-bit."""
    H, nh, nkv, hd, eps = cfg["r_hidden"], cfg["r_heads"], cfg["r_kv_heads"], cfg["r_head_dim"], cfg["r_eps"]
    w = {k: v.double() for k, v in w.items()}
    norm = lambda x, g: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * g
    T = len(ids)
    pos = torch.arange(T, dtype=torch.float64)[:, None, None]
    h = w["emb.weight"][torch.tensor(ids)]
    margin = torch.full((T,), float("inf"), dtype=torch.float64)    # how clear the closest routing decision at a place is
    for i in range(cfg["r_layers"]):
        p = f"blocks.{i}."
        x = norm(h, w[p + "n1.weight"])
        q = (x @ w[p + "q.weight"].T).view(T, nh, hd) * (1.0 + 0.01 * pos)
        k = (x @ w[p + "k.weight"].T).view(T, nkv, hd) * torch.cos(0.3 * pos)
        v = (x @ w[p + "v.weight"].T).view(T, nkv, hd)
        o = torch.zeros(T, nh, hd, dtype=torch.float64)
        for hh in range(nh):
            s = (q[:, hh] @ k[:, hh // (nh // nkv)].T) * hd ** -0.5
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            o[:, hh] = torch.softmax(s, -1) @ v[:, hh // (nh // nkv)]
        h = h + o.reshape(T, nh * hd) @ w[p + "o.weight"].T
        x = norm(h, w[p + "n2.weight"])
        pr = torch.softmax(x @ w[p + "router.weight"].T, -1)
        top = pr.argmax(-1)
        best2 = pr.topk(2, -1).values
        margin = torch.minimum(margin, best2[:, 0] - best2[:, 1])
        y = torch.zeros_like(h)
        for e in range(cfg["r_experts"]):
            g = x @ w[p + f"experts.{e}.g.weight"].T
            ye = ((g * torch.sigmoid(g)) * (x @ w[p + f"experts.{e}.u.weight"].T)) @ w[p + f"experts.{e}.d.weight"].T
            y += ye * (pr[:, e] * (top == e))[:, None]
        h = h + y
    return (norm(h, w["out_norm.weight"]) @ w["head.weight"].T).float(), margin.float()


@pytest.mark.parametrize("dtype,hd", [("float32", 24), ("bfloat16", 64)])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_around_the_library_attention(tmp_path, dtype, hd):
    """Parts of the test's own (a feed-forward that routes, a position encoding that is no rotation) are
    registered, built into a model with the library's attention, cache and step function, and stepped:
    prompts of unequal lengths, then token by token, against a plain whole-sequence computation.  In
    bfloat16 with a head size the tensor-core decode kernel takes, this is also the path on which that kernel
    must NOT rotate by itself."""
    import trapetum_b200 as tb
    _register_routed()
    cfg = {"architectures": ["TestRoutedLM"], "r_layers": 2, "r_hidden": 48, "r_heads": 3, "r_kv_heads": 1, "r_head_dim": hd,
           "r_inter": 80, "r_experts": 3, "r_vocab": 70, "r_eps": 1e-5}
    d = str(tmp_path / "routed")
    tb.write_random_model(d, cfg, 9, 0.15, 0.3)       # a seed whose routing decisions are clear for long
    # a router with random weights of this size is nearly undecided everywhere: make it decide
    from safetensors.torch import load_file, save_file
    stored = load_file(d + "/model.safetensors")
    for k in stored:
        if k.endswith("router.weight"):
            stored[k] = (stored[k].float() * 25.0).to(stored[k].dtype)
    save_file(stored, d + "/model.safetensors")
    pw = plain.load_folder(d)[1]
    model = tb.load_model(d, dtype)
    eng = tb.Engine(model, 64 * 6, max_slots=3)
    prompts = make_prompts(70, [33, 9, 20], seed=2)
    both = [_routed_plain(cfg, pw, p) for p in prompts]
    truth = [b[0] for b in both]
    # In bfloat16 a routing decision that is nearly a tie may fall the other way: that is another function, not
    # an error, and it changes every later place of its sequence through the keys and values.  So a sequence is
    # compared up to its first place whose closest decision is not clear in the 64-bit computation.
    clear = 0.0 if dtype == "float32" else 0.1
    upto = []
    for _, margin in both:
        unclear = (margin <= clear).nonzero()
        upto.append(int(unclear[0]) if len(unclear) else len(margin))
    tol = 2e-5 if dtype == "float32" else 4e-2
    s = eng.start(3)
    cut = [20, 4, 11]
    first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut])
    errs, o = [], 0
    for r in range(3):
        errs += [rel_l2(first[o + i], truth[r][i]) for i in range(min(cut[r], upto[r]))]
        o += cut[r]
    for t in range(5):
        out = eng.step(s, [[prompts[r][cut[r] + t]] for r in range(3)])
        errs += [rel_l2(out[r], truth[r][cut[r] + t]) for r in range(3) if cut[r] + t < upto[r]]
    eng.release(s)
    assert len(errs) >= 20, f"too few places with clear routing to say anything: {upto}"
    assert max(errs) < tol, sorted(errs)[-5:]


# ---------------------------------------------------------------------------
# The library's attention with biases and per-head norms of q and k: parameters, not a kernel edit
# ---------------------------------------------------------------------------
def _register_biased():
    from trapetum_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from trapetum_b200.config.base import _get

    @dataclass(frozen=True)
    class BiasedConfig:
        layers: int; hidden: int; heads: int; kv_heads: int; head_dim: int; inter: int; vocab: int; eps: float; window: int

        @classmethod
        def from_dict(cls, d):
            g = lambda k, t=int: _get(d, "b_" + k, t)
            return cls(g("layers"), g("hidden"), g("heads"), g("kv_heads"), g("head_dim"), g("inter"), g("vocab"),
                       g("eps", float), g("window"))

    def spec(c):
        norm = lambda n, size=c.hidden: PartSpec("rmsnorm", {"size": size, "eps": c.eps, "unit_offset": False, "weight": n})
        layers = tuple(LayerSpec(
            block=PartSpec("pre_norm", {"pre_mixer_norm": norm("n1.weight"), "pre_ffn_norm": norm("n2.weight")}),
            mixer=PartSpec("attention", {
                "hidden_size": c.hidden, "num_heads": c.heads, "num_kv_heads": c.kv_heads, "head_dim": c.head_dim,
                "scale": c.head_dim ** -0.5, "softcap": None, "window": c.window if i % 2 else None,
                "q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight",
                "bias": {"q": "q.bias", "k": "k.bias", "v": "v.bias", "o": "o.bias"},
                "q_norm": norm("q_norm.weight", c.head_dim), "k_norm": norm("k_norm.weight", c.head_dim),
                "position": PartSpec("rope", {"head_dim": c.head_dim, "theta": 1000.0, "rotary_dim": c.head_dim})}),
            feed_forward=PartSpec("gated_mlp", {"hidden_size": c.hidden, "intermediate_size": c.inter, "activation": "silu",
                                                "gate": "g.weight", "up": "u.weight", "down": "d.weight"}),
            prefix=f"blocks.{i}.") for i in range(c.layers))
        return ModelSpec(architecture="TestBiasedLM", hidden_size=c.hidden, vocab_size=c.vocab,
                         embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.hidden, "scale": 1.0,
                                                          "weight": "emb.weight"}),
                         layers=layers, schedule=tuple(ScheduleEntry(i) for i in range(c.layers)),
                         final_norm=norm("out_norm.weight"),
                         head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.hidden, "softcap": None,
                                                       "weight": "head.weight", "tied_to": None}),
                         max_positions=512)
    register_architecture("TestBiasedLM", BiasedConfig, spec)


def _biased_plain(cfg, w, ids, rnd=lambda x: x):
    """The biased, head-normed toy model, whole sequence, in 64-bit on the CPU."""
    nh, nkv, hd, eps, W = cfg["b_heads"], cfg["b_kv_heads"], cfg["b_head_dim"], cfg["b_eps"], cfg["b_window"]
    w = {k: v.double() for k, v in w.items()}
    norm = lambda x, g: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * g
    T = len(ids)
    h = w["emb.weight"][torch.tensor(ids)]
    for i in range(cfg["b_layers"]):
        p = f"blocks.{i}."
        x = rnd(norm(h, w[p + "n1.weight"]))
        q = rnd(norm(rnd(x @ w[p + "q.weight"].T + w[p + "q.bias"]).view(T, nh, hd), w[p + "q_norm.weight"]))
        k = rnd(norm(rnd(x @ w[p + "k.weight"].T + w[p + "k.bias"]).view(T, nkv, hd), w[p + "k_norm.weight"]))
        v = rnd(x @ w[p + "v.weight"].T + w[p + "v.bias"]).view(T, nkv, hd)
        q, k = rnd(plain.rope(q, torch.arange(T), 1000.0)), rnd(plain.rope(k, torch.arange(T), 1000.0))
        o = rnd(plain.attention(q, k, v, hd ** -0.5, None, W if i % 2 else None, rnd))
        h = h + o.reshape(T, nh * hd) @ w[p + "o.weight"].T + w[p + "o.bias"]
        x = rnd(norm(h, w[p + "n2.weight"]))
        g = rnd(x @ w[p + "g.weight"].T)
        h = h + rnd((g * torch.sigmoid(g)) * rnd(x @ w[p + "u.weight"].T)) @ w[p + "d.weight"].T
    return (rnd(norm(h, w["out_norm.weight"])) @ w["head.weight"].T).float()


@pytest.mark.parametrize("host", ["python", "native"])
@pytest.mark.parametrize("dtype,hd", [("float32", 24), ("bfloat16", 64), ("bfloat16", 32)])
def test_attention_with_biases_and_head_norms_is_a_matter_of_parameters(tmp_path, dtype, hd, host):
    """The library's attention part with a bias on each projection and an RMS norm on every query and key head:
    a model made of it is registered from here, built and stepped (prompts, then token by token, in a batch of
    unequal lengths) against a plain computation.  With a head size that the tensor-core decode kernel takes,
    the part must not hand that kernel its raw projection (the kernel's own prologue knows neither biases nor
    norms): it says so through ``fused_decode()``."""
    import trapetum_b200 as tb
    _register_biased()
    cfg = {"architectures": ["TestBiasedLM"], "b_layers": 2, "b_hidden": 64, "b_heads": 4, "b_kv_heads": 2, "b_head_dim": hd,
           "b_inter": 96, "b_vocab": 120, "b_eps": 1e-5, "b_window": 7}
    d = str(tmp_path / "biased")
    tb.write_random_model(d, cfg, 21, 0.2, 0.3)
    from safetensors.torch import load_file, save_file
    stored = load_file(d + "/model.safetensors")
    for k in stored:                                   # norm weights around 1, biases large enough to matter
        if "norm" in k or ".n1." in k or ".n2." in k:
            stored[k] = (1.0 + stored[k].float()).to(stored[k].dtype)
        if k.endswith(".bias"):
            stored[k] = (stored[k].float() * 3.0).to(stored[k].dtype)
    save_file(stored, d + "/model.safetensors")
    pw = plain.load_folder(d)[1]
    assert not any(b.mixer.fused_decode() for b in tb.load_model(d, dtype, host="python").blocks)
    model = tb.load_model(d, dtype, host=host)
    eng = tb.Engine(model, 64 * 6, max_slots=3)
    for g in eng.cache.groups:
        g.k.fill_(float("nan")); g.v.fill_(float("nan"))
    prompts = make_prompts(120, [40, 9, 23], seed=5)
    truth = [_biased_plain(cfg, pw, p) for p in prompts]
    if dtype == "float32":
        tol = [2e-5] * 3
    else:
        tol = [max(TOL["bfloat16"], 1.5 * max(rel_l2(a, b) for a, b in zip(_biased_plain(cfg, pw, p, plain.to_bf16), t)))
               for p, t in zip(prompts, truth)]
    cut = [28, 3, 12]
    s = eng.start(3)
    first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut])
    o = 0
    for r in range(3):
        worst = max(rel_l2(first[o + i], truth[r][i]) for i in range(cut[r]))
        assert worst <= tol[r], f"request {r} prompt: {worst:.3e} > {tol[r]:.2e}"
        o += cut[r]
    for t in range(6):
        out = eng.step(s, [[prompts[r][cut[r] + t]] for r in range(3)])
        for r in range(3):
            e = rel_l2(out[r], truth[r][cut[r] + t])
            assert e <= tol[r], f"request {r} token {cut[r] + t}: {e:.3e} > {tol[r]:.2e}"
    eng.release(s)
    # without biases and head norms the same part does hand the decode kernel its raw projection
    from trapetum_b200.config import load_config
    plain_mixer = tb.load_config(dict(TINY_A))[1].layers[0].mixer
    from trapetum_b200.parts import build_part
    m = build_part("mixer", plain_mixer, "model.layers.0.", _rt(torch.bfloat16))
    m.bind({n: torch.zeros(sp.shape, dtype=torch.bfloat16, device="cuda") for n, sp in m.tensor_specs().items()})
    assert m.fused_decode()


def test_a_state_of_another_dtype():
    from trapetum_b200.cache import Cache
    from trapetum_b200.parts import StateNeed
    c = Cache({0: StateNeed((3, 5), torch.bfloat16), 1: StateNeed((2,), torch.int32)}, {}, 64 * 4, torch.bfloat16, "cuda", 4)
    assert c.states[0].dtype == torch.bfloat16 and c.states[0].shape == (4, 3, 5) and c.states[1].dtype == torch.int32
    s = c.claim()
    c.view(0, 0).data[s].fill_(2.5)
    c.view(1, 1).data[s].fill_(7)
    c.release(s)
    assert c.claim() == s and float(c.states[0][s].abs().sum()) == 0.0 and int(c.states[1][s].sum()) == 0

"""The kernels at the layer sizes of Gemma-2-2B, 9B and 27B, two layers each, random weights: the engine in
bfloat16 and in true 32-bit against the plain implementation.  The tiny models never reach the tensor-core
tile sizes, the split-K paths or the 128- and 256-wide heads that the real sizes use.  2B keeps the real
vocabulary (256000); 9B and 27B use a smaller one so that the oracle's output product stays quick on a CPU.
27B has query_pre_attn_scalar (144) different from head_dim (128)."""
import pytest
import torch

import plain_gemma2 as plain
from conftest import decode_partition, TOL, bf16_budget, make_prompts, rel_l2, sharpen, within

pytestmark = pytest.mark.gpu

BASE = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": 2,
    "rope_theta": 10000.0, "sliding_window": 96, "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0,
    "rms_norm_eps": 1e-6, "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True,
    "max_position_embeddings": 8192,
}
SHAPES = {
    "2b": dict(BASE, hidden_size=2304, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
               intermediate_size=9216, vocab_size=256000, query_pre_attn_scalar=256),
    "9b": dict(BASE, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               intermediate_size=14336, vocab_size=32000, query_pre_attn_scalar=256),
    "27b": dict(BASE, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                intermediate_size=36864, vocab_size=32000, query_pre_attn_scalar=144),
}
SEEDS = {"2b": 2, "9b": 3, "27b": 4}
BF16_TOL = {}        # shape name -> bfloat16 tolerance per prompt


def tolerances(shape, dtype, n=3):
    return [TOL["float32"]] * n if dtype == "float32" else BF16_TOL[shape]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """shape name -> (folder, config, weights, prompts, oracle logits), made on first use."""
    import trapetum_b200 as tb
    made = {}

    def get(name):
        if name not in made:
            d = str(tmp_path_factory.mktemp("real_" + name))
            tb.write_random_model(d, SHAPES[name], seed=SEEDS[name], std=0.02, norm_std=0.1)
            sharpen(d, 2.0)
            # float64: with inner sizes of up to 36864 the oracle's own rounding in float32 would be as large
            # as the 32-bit engine's, and the oracle has to be the more exact of the two
            cfg, w = plain.load_folder(d, dtype=torch.float64)
            prompts = make_prompts(cfg["vocab_size"], [150, 37, 220], seed=4)
            made[name] = (d, cfg, w, prompts, [plain.forward(cfg, w, p) for p in prompts])
            BF16_TOL[name] = [bf16_budget(cfg, w, [p]) for p in prompts]      # per sequence, from the oracle alone
        return made[name]
    return get


@pytest.mark.parametrize("variant", ["as chosen", "stream and pairs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["2b", "9b", "27b"])
def test_logits_at_real_layer_sizes(models, shape, dtype, variant):
    """Three unequal prompts, then one token each.  Contexts this short are cut into pieces whatever their
    lengths, and prompts this short run their products on single SMs; the second run deals the pages out as one
    stream and sends the products to pairs of SMs, as the library does for long uneven batches and long prompts."""
    from trapetum_b200.csrc import ops
    if variant != "as chosen" and dtype == "float32":
        pytest.skip("the 32-bit path has one attention kernel and one product kernel")
    was = ops.gemm_tc_set_pair(1 if variant != "as chosen" else 2)
    try:
        with decode_partition("stream" if variant != "as chosen" else None):
            _logits_at_real_layer_sizes(models, shape, dtype)
    finally:
        ops.gemm_tc_set_pair(was)


def _logits_at_real_layer_sizes(models, shape, dtype):
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    folder, cfg, w, prompts, want = models(shape)
    tol = tolerances(shape, dtype)
    model = tb.load_model(folder, dtype)
    eng = tb.Engine(model, max_tokens=64 * 12)
    for g in eng.cache.groups:
        g.k.fill_(float("nan")); g.v.fill_(float("nan"))
    # a first step of three unequal prompts (their last 20 tokens held back), then one token each
    cut = [len(p) - 20 for p in prompts]
    s = eng.start(3)
    got = [[] for _ in prompts]
    first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [[0, c // 2, c - 1] for c in cut])
    for r, c in enumerate(cut):
        for k, i in enumerate([0, c // 2, c - 1]):
            within(rel_l2(first[3 * r + k], want[r][i]), tol[r], dtype, f"{shape} sizes: prompt {r} position {i}")
    for t in range(20):
        out = eng.step(s, [[p[c + t]] for p, c in zip(prompts, cut)])
        assert torch.isfinite(out).all()
        for r, c in enumerate(cut):
            within(rel_l2(out[r], want[r][c + t]), tol[r], dtype, f"{shape} sizes: request {r} decoded token {t}")
    eng.release(s)
    torch.cuda.synchronize()
    assert ops.kernel_errors() == {}


def _equal_batch_and_batch_of_one(eng, prompts, want, n_equal, n_prefill, tol, dtype, what):
    """Two sequences of the same length, then one sequence alone: prompt in one step, the rest token by token.
    Decode steps of equal lengths (and of one sequence) cut every sequence into the same number of pieces (the
    attention kernel's *split* partition, which also rotates q and k and appends to the cache by itself); from
    its second occurrence on the step runs as a replayed graph."""
    from trapetum_b200.engine.engine import uneven_lengths
    for g in eng.cache.groups:
        g.k.fill_(float("nan")); g.v.fill_(float("nan"))
    for rows in ([0, 1], [1]):
        seqs = [prompts[r][:n_equal] for r in rows]
        s = eng.start(len(rows))
        first = eng.step(s, [q[:n_prefill] for q in seqs], [[n_prefill - 1]] * len(rows))
        for i, r in enumerate(rows):
            within(rel_l2(first[i], want[r][n_prefill - 1]), tol[r], dtype, f"{what}: batch {rows}, request {r}, prompt's end")
        for t in range(n_prefill, n_equal):
            assert not uneven_lengths([t + 1] * len(rows))
            out = eng.step(s, [[q[t]] for q in seqs])
            assert torch.isfinite(out).all()
            for i, r in enumerate(rows):
                within(rel_l2(out[i], want[r][t]), tol[r], dtype, f"{what}: batch {rows}, request {r}, token {t}")
        eng.release(s)
    assert eng.graphs_captured >= 1                                       # steps did run as replayed graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["2b", "9b", "27b"])
def test_equal_lengths_and_batch_of_one_at_real_layer_sizes(models, shape, dtype):
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    folder, cfg, w, prompts, want = models(shape)
    tol = tolerances(shape, dtype)
    tol = [tol[0], tol[2]]
    eng = tb.Engine(tb.load_model(folder, dtype), max_tokens=64 * 8)
    # requests 0 and 2 (150 and 220 tokens), both cut to 150: a causal model's logits at a place do not
    # depend on what follows it, so the oracle's logits of the longer one hold for its first 150 tokens
    _equal_batch_and_batch_of_one(eng, [prompts[0], prompts[2]], [want[0], want[2]], 150, 126, tol, dtype, f"{shape} sizes")
    torch.cuda.synchronize()
    assert ops.kernel_errors() == {}


@pytest.mark.parametrize("lens", [[3000, 2900, 3100, 2950, 3050, 3000, 2980, 3020], [6000, 70, 300, 64, 1500, 9, 640, 1]])
def test_decoding_repeats_bit_for_bit_over_long_contexts(models, lens):
    """Decode steps over contexts of thousands of tokens (cache filled with random keys and values), once with
    lengths that are nearly equal (the split partition) and once with lengths that differ widely (the stream
    partition).  The attention kernel's pieces are counted with atomics and folded by whichever CTA finishes
    last: the result must not depend on that, so two engines with the same cache content must give the same
    bits, step after step."""
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    from trapetum_b200.engine.engine import uneven_lengths
    folder, cfg, _, _, _ = models("2b")
    model = tb.load_model(folder, "bfloat16")
    B, steps = len(lens), 12
    outs = []
    for run in range(2):
        eng = tb.Engine(model, max_tokens=sum(-(-(n + steps) // 64) * 64 for n in lens), max_slots=B)
        gen = torch.Generator(device="cuda").manual_seed(11)
        for g in eng.cache.groups:
            g.k.copy_(torch.randn(g.k.shape, device="cuda", generator=gen).mul_(0.5))
            g.v.copy_(torch.randn(g.v.shape, device="cuda", generator=gen).mul_(0.5))
        slots = eng.start(B)
        eng.cache.grow({s: n for s, n in zip(slots, lens)})
        toks = torch.randint(0, cfg["vocab_size"], (steps, B), generator=torch.Generator().manual_seed(5)).tolist()
        got = []
        for t in range(steps):
            got.append(eng.step(slots, [[x] for x in toks[t]]).clone())
        torch.cuda.synchronize()
        outs.append(torch.stack(got))
        eng.release(slots)
        del eng
    assert uneven_lengths(lens) == (min(lens) < 100)
    assert torch.isfinite(outs[0]).all()
    assert torch.equal(outs[0], outs[1])
    assert ops.kernel_errors() == {}


MID = dict(BASE, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512,
           vocab_size=1000, query_pre_attn_scalar=64, sliding_window=200)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_through_the_tensor_core_attention(tmp_path_factory, dtype):
    """Prompts of many key blocks (900 and 333 tokens, a window of 200 on the even layers) through a model whose
    head size (64) takes the tcgen05 prefill kernel and the tensor-core decode kernel, then eight tokens one by
    one: logits at the first position, around the window's edge, in the middle and at the end."""
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    d = str(tmp_path_factory.mktemp("mid"))
    tb.write_random_model(d, MID, seed=9, std=0.05, norm_std=0.1)
    sharpen(d, 2.0)
    cfg, w = plain.load_folder(d, dtype=torch.float64)
    prompts = make_prompts(cfg["vocab_size"], [908, 341], seed=6)
    want = [plain.forward(cfg, w, p) for p in prompts]
    tol = [TOL["float32"]] * 2 if dtype == "float32" else [bf16_budget(cfg, w, [p]) for p in prompts]
    model = tb.load_model(d, dtype)
    eng = tb.Engine(model, max_tokens=64 * 22)
    for g in eng.cache.groups:
        g.k.fill_(float("nan")); g.v.fill_(float("nan"))
    cut = [len(p) - 8 for p in prompts]
    places = [[0, 127, 128, 199, 200, 201, c // 2, c - 1] for c in cut]
    s = eng.start(2)
    first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], places)
    k = 0
    for r in range(2):
        for i in places[r]:
            within(rel_l2(first[k], want[r][i]), tol[r], dtype, f"head size 64: prompt {r} position {i}")
            k += 1
    for t in range(8):
        out = eng.step(s, [[p[c + t]] for p, c in zip(prompts, cut)])
        for r, c in enumerate(cut):
            within(rel_l2(out[r], want[r][c + t]), tol[r], dtype, f"head size 64: request {r} decoded token {t}")
    eng.release(s)
    # equal lengths and a batch of one, across the border between two length buckets (256 tokens)
    eng2 = tb.Engine(model, max_tokens=64 * 12)
    _equal_batch_and_batch_of_one(eng2, prompts, want, 300, 236, tol, dtype, "head size 64")
    assert eng2.graphs_captured >= 2                                       # two length buckets, a graph each
    torch.cuda.synchronize()
    assert ops.kernel_errors() == {}


class _LazyWeights:
    """name -> tensor, read from the folder and widened when asked for and not kept: the plain implementation
    walks a whole 26-layer model without ever holding more than one matrix in 64-bit."""

    def __init__(self, folder, dtype):
        from safetensors import safe_open
        self.f = safe_open(folder + "/model.safetensors", framework="pt")
        self.names, self.dtype = set(self.f.keys()), dtype

    def __getitem__(self, name):
        return self.f.get_tensor(name).to(self.dtype)

    def __contains__(self, name):
        return name in self.names

    def get(self, name, default=None):
        return self[name] if name in self.names else default


def test_whole_2b_model_against_the_plain_implementation(tmp_path_factory):
    """All 26 layers at Gemma-2-2B's sizes with its real vocabulary and the weights as the generator makes
    them: a 64-token sequence, its first 48 tokens as a prompt and the rest one by one, in bfloat16 and in
    32-bit, against the plain implementation in 64-bit on every position.  The engine's model is made on the
    device (tb.random_model); the oracle reads the folder that write_random_model writes for the same seed."""
    import json
    import trapetum_b200 as tb
    from trapetum_b200.csrc import ops
    cfg = dict(SHAPES["2b"], num_hidden_layers=26, sliding_window=32)
    d = str(tmp_path_factory.mktemp("whole_2b"))
    tb.write_random_model(d, cfg, seed=2, std=0.02, norm_std=0.1)
    ids = make_prompts(cfg["vocab_size"], [64], seed=12)[0]
    want = plain.forward(json.load(open(d + "/config.json")), _LazyWeights(d, torch.float64), ids)
    for dtype in ("bfloat16", "float32"):
        model = tb.random_model(cfg, 2, 0.02, 0.1, dtype)
        eng = tb.Engine(model, max_tokens=128)
        for g in eng.cache.groups:
            g.k.fill_(float("nan")); g.v.fill_(float("nan"))
        s = eng.start(1)
        got = [eng.step(s, [ids[:48]], [list(range(48))])]
        for t in range(48, 64):
            got.append(eng.step(s, [[ids[t]]]))
        eng.release(s)
        got = torch.cat(got)
        assert torch.isfinite(got).all()
        within(max(rel_l2(got[i], want[i]) for i in range(64)), TOL[dtype], dtype, "whole 2B model, 64 tokens")
        if dtype == "float32":
            assert (got.cpu().argmax(-1) == want.argmax(-1)).all()
        del eng, model
        torch.cuda.empty_cache()
    assert ops.kernel_errors() == {}

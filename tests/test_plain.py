"""The plain implementation checked against its own formulas (no GPU): it is the oracle of the
GPU tests, so each of its parts is pinned here by hand-computed values and by properties."""
import math

import pytest
import torch

import plain_gemma2 as plain
from conftest import TINY_A, TINY_B, TINY_C, make_prompts


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([0.5, -0.25])
    y = plain.rmsnorm(x, w, 1e-6)
    r = 1.0 / math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(y, torch.tensor([[3 * r * 1.5, 4 * r * 0.75]]), atol=1e-6)


def test_rope_by_hand_and_relative():
    x = torch.zeros(2, 1, 4)
    x[:, 0, :] = torch.tensor([1.0, 2.0, 3.0, 4.0])
    y = plain.rope(x, torch.tensor([0, 3]), 100.0)
    assert torch.allclose(y[0], x[0])                                   # position 0: unchanged
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)                                 # angles of pairs (0,2) and (1,3)
    want = torch.tensor([1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                         3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)])
    assert torch.allclose(y[1, 0], want, atol=1e-6)
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    s = lambda i, j: float((plain.rope(q, torch.tensor([i]), 1e4) * plain.rope(k, torch.tensor([j]), 1e4)).sum())
    assert s(5, 2) == pytest.approx(s(13, 10), abs=1e-5)


def test_visibility():
    assert plain.visible(5, 5, 3) and plain.visible(5, 3, 3) and not plain.visible(5, 2, 3)
    assert not plain.visible(2, 3, None) and plain.visible(100, 0, None)


def test_attention_by_hand():
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]]])          # T=2, one head
    k = torch.tensor([[[1.0, 1.0]], [[3.0, 1.0]]])
    v = torch.tensor([[[1.0, 10.0]], [[2.0, 20.0]]])
    o = plain.attention(q, k, v, scale=0.5, cap=None, window=None)
    assert torch.allclose(o[0, 0], v[0, 0])                  # the first query sees only itself
    s = torch.tensor([0.5 * 2.0, 0.5 * 2.0])                 # second query: scores 1, 1
    p = torch.softmax(s, 0)
    assert torch.allclose(o[1, 0], p[0] * v[0, 0] + p[1] * v[1, 0])
    capped = plain.attention(q * 100, k, v, scale=0.5, cap=2.0, window=None)
    s = 2.0 * torch.tanh(torch.tensor([0.0 * 50, 200 * 0.5 / 2.0]))    # 0 and 2*tanh(50)
    s = 2.0 * torch.tanh(torch.tensor([(0 * 1 + 200 * 1) * 0.5 / 2.0, (0 * 3 + 200 * 1) * 0.5 / 2.0]))
    p = torch.softmax(s, 0)
    assert torch.allclose(capped[1, 0], p[0] * v[0, 0] + p[1] * v[1, 0], atol=1e-5)
    windowed = plain.attention(q, k, v, scale=0.5, cap=None, window=1)
    assert torch.allclose(windowed[1, 0], v[1, 0])           # a window of one: only itself


def test_gqa_head_mapping():
    T, nh, nkv, hd = 3, 4, 2, 4
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    o = plain.attention(q, k, v, 0.5, None, None)
    for h in range(nh):
        alone = plain.attention(q[:, h:h + 1], k[:, h // 2:h // 2 + 1], v[:, h // 2:h // 2 + 1], 0.5, None, None)
        assert torch.allclose(o[:, h], alone[:, 0], atol=1e-6)


def test_gelu_and_feed_forward():
    g = torch.tensor([0.0, 1.0, -2.0])
    want = [0.0, 0.5 * (1 + math.tanh(0.7978845608 * 1.044715)), -1.0 * (1 + math.tanh(0.7978845608 * (-2 - 0.044715 * 8)))]
    assert torch.allclose(plain.gelu_tanh(g), torch.tensor(want), atol=1e-6)
    x = torch.randn(2, 3); wg, wu, wd = torch.randn(5, 3), torch.randn(5, 3), torch.randn(3, 5)
    assert torch.allclose(plain.feed_forward(x, wg, wu, wd), (plain.gelu_tanh(x @ wg.T) * (x @ wu.T)) @ wd.T)


def _weights(cfg, seed, std=0.05, nstd=0.2):
    import trapetum_b200 as tb
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        tb.write_random_model(d, cfg, seed, std, nstd)
        return plain.load_folder(d)


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C])
def test_causality_and_shapes(cfg):
    c, w = _weights(cfg, 0)
    ids = make_prompts(cfg["vocab_size"], [20], 1)[0]
    full = plain.forward(c, w, ids)
    assert full.shape == (20, cfg["vocab_size"]) and torch.isfinite(full).all()
    part = plain.forward(c, w, ids[:13])
    assert torch.allclose(full[:13], part, atol=1e-5)            # later tokens change nothing earlier
    cap = cfg.get("final_logit_softcapping")
    if cap:
        assert float(full.abs().max()) <= cap


def test_window_bites_only_on_sliding_layers():
    c, w = _weights(TINY_A, 0, std=0.2)
    ids = make_prompts(256, [24], 2)[0]
    wide = dict(c, sliding_window=1000)
    a, b = plain.forward(c, w, ids), plain.forward(wide, w, ids)
    assert torch.allclose(a[:8], b[:8], atol=1e-6)               # within the window nothing differs
    assert not torch.allclose(a[8:], b[8:], atol=1e-4)           # beyond it the sliding layers see less
    assert plain.layer_is_sliding(c, 0) and not plain.layer_is_sliding(c, 1)


def test_float64_agrees_with_float32():
    c, w = _weights(TINY_B, 1)
    ids = make_prompts(384, [17], 3)[0]
    w64 = {k: v.double() for k, v in w.items()}
    a, b = plain.forward(c, w, ids), plain.forward(c, w64, ids)
    assert float((a.double() - b).norm() / b.norm()) < 1e-5


def test_schedule_with_a_repeated_layer_and_a_shared_cache():
    c, w = _weights(TINY_A, 0, std=0.1)
    ids = make_prompts(256, [9], 4)[0]
    base = plain.forward(c, w, ids)
    twice = plain.forward(c, w, ids, schedule=[(0, None), (1, None), (0, None)])
    shared = plain.forward(c, w, ids, schedule=[(0, None), (1, None), (0, 0)])
    assert not torch.allclose(base, twice, atol=1e-4) and not torch.allclose(twice, shared, atol=1e-4)


def test_choosing_tokens():
    assert plain.greedy(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1                 # first of the tied maxima
    l = torch.tensor([2.0, -1.0, 0.5, 4.0])
    out = plain.repetition_penalty(l, [0, 1, 1, -1], 2.0)
    assert out.tolist() == [1.0, -2.0, 0.5, 4.0]
    assert plain.repetition_penalty(l, [0], 1.0).tolist() == l.tolist()
    p = plain.nucleus(torch.tensor([0.0, math.log(2.0), math.log(4.0), math.log(1.0)]), 1.0, 0.7)
    # probabilities 1/8, 2/8, 4/8, 1/8: 4/8 alone is below 0.7, with 2/8 it passes
    assert p.tolist() == pytest.approx([0.0, 1 / 3, 2 / 3, 0.0])
    assert plain.nucleus(torch.tensor([0.0, 0.0]), 0.5, 1.0).tolist() == pytest.approx([0.5, 0.5])


def test_greedy_generation_stops():
    c, w = _weights(TINY_A, 0)
    out = plain.generate_greedy(c, w, [1, 2, 3], 5)
    assert len(out) == 5
    assert plain.generate_greedy(c, w, [1, 2, 3], 5, stop_ids=[out[2]]) == out[:out.index(out[2])]


def test_parts_against_the_outputs_of_the_reference_s_own_cuda_operators():
    """tests/golden/reference_ops.json holds what runtime/cuda/codebook_gemv.cu (compiled unchanged, run on a
    B200 by tests/golden/make_reference_ops_golden.py) computes on small float16 cases: RMS norm, rotation,
    one-query attention with and without the soft cap, GeGLU, residual sum, greedy choice.  The plain
    implementation's functions must give the same numbers to float16 accuracy."""
    import json
    import os
    from reference_ops_check import check_all
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_ops.json")
    with open(path) as f:
        stored = json.load(f)["outputs"]
    ref = {k: (v if isinstance(v, int) else torch.tensor(v["values"], dtype=torch.float32).reshape(v["shape"]))
           for k, v in stored.items()}
    assert check_all(ref) == 10

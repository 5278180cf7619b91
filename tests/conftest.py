"""Shared pieces of the tests: the tiny configurations, model folders made in a temporary
place, and the error measures."""
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


def _cfg(**kw):
    base = {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "hidden_activation": "gelu_pytorch_tanh",
            "tie_word_embeddings": True, "max_position_embeddings": 8192}
    base.update(kw)
    return base


# Two tiny configurations that differ in every size and option, plus a third for what both share.
TINY_A = _cfg(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=128, vocab_size=256, rope_theta=10000.0, sliding_window=8, query_pre_attn_scalar=16,
              attn_logit_softcapping=50.0, final_logit_softcapping=30.0, rms_norm_eps=1e-6)
TINY_B = _cfg(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
              intermediate_size=160, vocab_size=384, rope_theta=1000.0, sliding_window=16, query_pre_attn_scalar=32,
              attn_logit_softcapping=None, final_logit_softcapping=15.0, rms_norm_eps=1e-5)
# query_pre_attn_scalar != head_dim, no final cap, as many kv heads as heads, a window that never bites
# a short prompt but does bite a long one, one layer more than B, a vocabulary and widths that are no
# power of two and not multiples of 8 (so the bfloat16 path must take its FMA fallback for some products).
TINY_C = _cfg(num_hidden_layers=4, hidden_size=72, num_attention_heads=3, num_key_value_heads=3, head_dim=48,
              intermediate_size=100, vocab_size=301, rope_theta=50000.0, sliding_window=70, query_pre_attn_scalar=24,
              attn_logit_softcapping=20.0, final_logit_softcapping=None, rms_norm_eps=1e-4)

# name -> (config, seed, std of matrices, std of norm weights, sharpening factor).  The factor is
# chosen so that attention scores have a spread of about 1.5 in every model: peaked enough that a
# wrong or missing key shows in the logits, not so peaked that 16-bit rounding alone flips them.
TINY = {"A": (TINY_A, 0, 0.02, 0.1, 8.0), "B": (TINY_B, 1, 0.03, 0.2, 4.0), "C": (TINY_C, 5, 0.05, 0.3, 2.5)}

# Tolerances on logits against the plain implementation (relative L2 over a position's logits,
# the reference's measure: runtime/src/bin/model.rs:131-139).  float32: rounding only.  bfloat16:
# 2e-2 for models with weights of N(0, 0.02) to N(0, 0.05); where a test sharpens attention on purpose,
# 16-bit storage alone costs more, and the budget is sized per model by bf16_budget() below.
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


BUDGET_FACTOR = 1.5


def bf16_budget(cfg, w, prompts, schedule=None) -> float:
    """The bfloat16 budget for a model: one and a half times the worst per-position error that the
    plain implementation itself shows when it rounds its stored activations to bfloat16
    (plain_gemma2.forward(rnd=to_bf16)), and never below TOL["bfloat16"].  It is computed from the
    oracle alone, before the engine runs."""
    import plain_gemma2 as plain
    worst = 0.0
    for p in prompts:
        exact = plain.forward(cfg, w, p, schedule)
        rounded = plain.forward(cfg, w, p, schedule, rnd=plain.to_bf16)
        worst = max(worst, max(rel_l2(rounded[i], exact[i]) for i in range(len(p))))
    return max(TOL["bfloat16"], BUDGET_FACTOR * worst)


_SEQ_BUDGET = {}


def seq_tolerance(key, cfg, w, ids, dtype: str, schedule=None) -> float:
    """The tolerance for the logits of ONE sequence: float32, rounding only; bfloat16, the budget that the
    oracle gives for this very sequence (where on a sequence 16-bit storage costs most differs from sequence
    to sequence, so a budget taken on other prompts would be too wide for some and too narrow for others).
    ``key`` names the model; results are kept."""
    if dtype == "float32":
        return TOL["float32"]
    k = (key, tuple(ids), None if schedule is None else tuple(schedule))
    if k not in _SEQ_BUDGET:
        _SEQ_BUDGET[k] = bf16_budget(cfg, w, [list(ids)], schedule)
    return _SEQ_BUDGET[k]


MEASURED = []          # (what, dtype, worst error, tolerance) of every logits comparison of the run


def within(worst: float, tol: float, dtype: str, what: str) -> None:
    """Assert that a measured error keeps its tolerance; the message and the run's summary show both, so
    that a tolerance far above what is measured is seen as well as one that is broken."""
    MEASURED.append((what, dtype, worst, tol))
    assert worst <= tol, f"{what} [{dtype}]: worst relative L2 error {worst:.3e} > tolerance {tol:.2e}"


def pytest_terminal_summary(terminalreporter):
    if not MEASURED:
        return
    tr = terminalreporter
    tr.write_line("")
    tr.write_line("logits against the plain implementation: worst measured error / tolerance, per dtype")
    for dtype in sorted({m[1] for m in MEASURED}):
        rows = sorted((m for m in MEASURED if m[1] == dtype), key=lambda m: -m[2] / m[3])
        ratios = [m[2] / m[3] for m in rows]
        tr.write_line(f"  {dtype}: {len(rows)} comparisons, error/tolerance max {ratios[0]:.3f}, "
                      f"median {ratios[len(ratios) // 2]:.3f}")
        for what, _, worst, tol in rows[:6]:
            tr.write_line(f"    {worst:.3e} / {tol:.2e}  {what}")


def rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def sharpen(folder: str, factor: float = 8.0) -> None:
    """Scale the query and key projections so that attention is peaked: with weights of
    N(0, 0.02) every softmax is nearly flat and a wrong key would barely move the logits."""
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    w = load_file(path)
    for k in list(w):
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            w[k] = (w[k].float() * factor).to(w[k].dtype)
    save_file(w, path)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (random weights, sharpened attention)."""
    import trapetum_b200 as tb
    out = {}
    for name, (cfg, seed, std, nstd, factor) in TINY.items():
        d = str(tmp_path_factory.mktemp("tiny" + name))
        tb.write_random_model(d, cfg, seed, std, nstd)
        sharpen(d, factor)
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_folders):
    import plain_gemma2 as plain
    return {name: plain.load_folder(d) for name, d in model_folders.items()}


@pytest.fixture(scope="session")
def tolerance_of(plain_models):
    """(model name, token ids, dtype) -> tolerance for that sequence's logits on the sharpened tiny models."""
    def get(name, ids, dtype):
        cfg, w = plain_models[name]
        return seq_tolerance(name, cfg, w, ids, dtype)
    return get


def make_prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


import contextlib


@contextlib.contextmanager
def decode_partition(mode):
    """Decode attention's partition forced on both hosts ("split", "stream"; None leaves the choice to the library)
    for engines made inside the block."""
    from trapetum_b200 import native
    from trapetum_b200.csrc import ops
    was_py = ops.set_decode_partition(mode)
    was_native = native.set_decode_partition(mode)
    try:
        yield
    finally:
        ops.set_decode_partition(was_py)
        native.set_decode_partition(was_native)

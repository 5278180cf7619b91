"""The comparison of the plain implementation's functions with the outputs of the reference's own CUDA
operators (runtime/cuda/codebook_gemv.cu), shared by the CPU test on stored outputs and the GPU test on
live ones.  The reference computes in float16 with 32-bit sums; the tolerance is that of float16 storage."""
import math
import os
import sys

import torch

import plain_gemma2 as plain

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from reference_ops_cases import ATTN, inputs  # noqa: E402

F16 = 2.0 ** -10            # half a unit in the last place of a float16 is 2^-11 of the value


def close(got: torch.Tensor, want: torch.Tensor, what: str, ulps: float = 2.0) -> None:
    """Element-wise: within ``ulps`` float16 roundings of the value, or of the largest value for entries
    that cancel."""
    got, want = got.double().reshape(-1), want.double().reshape(-1)
    bound = ulps * F16 * torch.maximum(want.abs(), 0.05 * want.abs().max())
    bad = (got - want).abs() > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} of {got.numel()} values differ, worst " \
                          f"{float(((got - want).abs() / bound).max()):.2f} times the float16 bound"


def check_all(ref: dict) -> int:
    """``ref``: case name -> the reference's output (float32 tensor, or an int for argmax)."""
    c = inputs()
    f = lambda t: t.float()
    x, w = f(c["rmsnorm"]["x"]), c["rmsnorm"]["w"].float()
    close(ref["rmsnorm"], plain.rmsnorm(x, w, c["rmsnorm"]["eps"]), "rmsnorm against op_rmsnorm")
    for name in ("rope", "rope_far"):
        x = f(c[name]["x"])
        want = plain.rope(x[None], torch.tensor([c[name]["pos"]]), c[name]["theta"])[0]
        # at position 8000 the 32-bit angle itself is only good to about 1e-3: allow for it there
        close(ref[name], want, f"{name} against op_rope", ulps=2.0 if name == "rope" else 8.0)
    for name, nh, nkv, hd, n, cap in ATTN:
        q, k, v = f(c[name]["q"]), f(c[name]["k"]), f(c[name]["v"])
        # the reference serves one query over n keys; the plain function is causal over whole sequences,
        # so the query becomes the last of n rows (the rows before it do not matter)
        qs = torch.zeros(n, nh, hd)
        qs[-1] = q
        want = plain.attention(qs, k, v, 1.0 / math.sqrt(hd), cap or None, None)[-1]
        close(ref[name], want, f"{name} against op_attn")
    g, u = c["gelu_mul"]["gate"], c["gelu_mul"]["up"]
    close(ref["gelu_mul"], plain.gelu_tanh(g) * u, "gelu_tanh * up against op_gelu_mul")
    close(ref["resadd_h"], f(c["resadd_h"]["h"]) + f(c["resadd_h"]["d"]), "residual sum against op_resadd_h", ulps=1.0)
    assert ref["argmax"] == plain.greedy(c["argmax"]["logits"]) == 77
    return 5 + len(ATTN) + 2

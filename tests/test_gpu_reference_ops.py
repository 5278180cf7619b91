"""The reference's own CUDA operators, run live, against the plain implementation and against this
library's kernels.  The operators come from runtime/cuda/codebook_gemv.cu of neuralboot/trapetum, compiled
unchanged for sm_100a into baseline/_ref/ by tests/golden/make_reference_ops_golden.py (that folder is not
committed: the test is skipped where neither the compiled library nor the reference's source is at hand).
Small cases only: one sequence, at most 300 keys, head sizes that are powers of two."""
import math
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))


@pytest.fixture(scope="module")
def reference_outputs():
    import make_reference_ops_golden as maker
    try:
        path = maker.build(os.environ.get("TRAPETUM_REFERENCE", ""))
    except (FileNotFoundError, OSError) as e:
        pytest.skip(f"the reference's kernel file is not at hand: {e}")
    return maker.run_all(maker.load(path))


def test_plain_implementation_against_the_reference_s_operators(reference_outputs):
    from reference_ops_check import check_all
    assert check_all(reference_outputs) == 10


def test_this_library_s_kernels_against_the_reference_s_operators(reference_outputs):
    """The same cases through this library's kernels (bfloat16 has three bits less than the reference's
    float16, so the float32 kernels are used on the float16 values)."""
    from reference_ops_cases import ATTN, inputs
    from reference_ops_check import close
    from trapetum_b200.csrc import ops
    c = inputs()
    x = c["rmsnorm"]["x"].float().cuda()[None]
    got = ops.rmsnorm(x, c["rmsnorm"]["w"].float().cuda(), c["rmsnorm"]["eps"], 1.0, torch.float32)[0]
    close(got.cpu(), reference_outputs["rmsnorm"], "rmsnorm kernel against op_rmsnorm")
    for name, nh, nkv, hd, n, cap in ATTN:
        q = c[name]["q"].float().cuda().reshape(1, nh * hd)
        pages = (n + 63) // 64
        kp = torch.zeros(pages, nkv, 64, hd, device="cuda")
        vp = torch.zeros_like(kp)
        for t in range(n):
            kp[t // 64, :, t % 64] = c[name]["k"][t].float().cuda()
            vp[t // 64, :, t % 64] = c[name]["v"][t].float().cuda()
        table = torch.arange(pages, dtype=torch.int32, device="cuda")[None]
        la = torch.tensor([n], dtype=torch.int32, device="cuda")
        got = ops.attn_decode_simt(q, kp, vp, table, la, nh, nkv, hd, 1.0 / math.sqrt(hd), cap, 0, 0, 2)
        close(got.cpu().reshape(nh, hd), reference_outputs[name], f"decode attention kernel against op_attn ({name})")
    a = c["argmax"]["logits"].cuda()[None]
    assert int(ops.argmax(a)[0]) == reference_outputs["argmax"] == 77

"""The decode attention entry point that allocates nothing (attention_decode_noalloc.h), called the way
a C program would call it: through the exported symbol, with a caller-owned output buffer.

Who this is for: callers that cannot allocate device memory at call time, such as a program that got a
fixed slice of device memory at start-up, or a latency-bound loop that cannot afford cudaMalloc's
synchronisation.  Its results must equal those of the ordinary entry point, whose scratch the caller
allocates, on consecutive calls that reuse the built-in scratch.  This file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
PAGE = 64


def _paged(lens, nkv, hd, n_pages, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    kp = (torch.randn(n_pages, nkv, PAGE, hd, device="cuda", generator=g) * 0.5).bfloat16()
    vp = (torch.randn(n_pages, nkv, PAGE, hd, device="cuda", generator=g) * 0.5).bfloat16()
    width = max((n + PAGE - 1) // PAGE for n in lens)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    for b, n in enumerate(lens):
        for pg in range((n + PAGE - 1) // PAGE):
            table[b, pg] = perm.pop()
    return kp, vp, table.cuda()


def _call_noalloc(ops, lib, q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, splits):
    """Fill the argument block by hand and call the exported C symbol; the output buffer is the caller's."""
    out = torch.empty((q.shape[0], nh * hd), dtype=q.dtype, device=q.device)
    a = ops._DecodeArgs()
    a.q = q.data_ptr(); a.q_stride = q.stride(0)
    a.k_pool = kp.data_ptr(); a.v_pool = vp.data_ptr()
    a.page_table = table.data_ptr(); a.pt_stride = table.stride(0)
    a.len_after = la.data_ptr(); a.out = out.data_ptr(); a.partial = None
    a.n_heads = nh; a.n_kv_heads = nkv; a.hd = hd; a.page_rows = PAGE
    a.ring_rows = ring; a.window = window; a.n_splits = splits
    a.scale = scale; a.cap = cap
    fn = lib.tb_attn_decode_noalloc
    fn.restype = ctypes.c_int
    status = fn(ctypes.byref(a), ctypes.c_int(ops.code(q.dtype)), ctypes.c_int(q.shape[0]),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return status, out


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from trapetum_b200.csrc import build, ops
    lib = build.load("attention_decode")
    nh, nkv, hd = 8, 4, 256
    scale = 1.0 / math.sqrt(hd)
    # two calls in a row with different lengths, splits and windows: the second finds the first one's
    # partials in the shared scratch and must not be disturbed by them
    for lens, splits, window, cap, seed in (([700, 64, 1, 333], 5, 0, 50.0, 1), ([90, 513, 260, 128], 3, 256, 0.0, 2)):
        ring = ((window + PAGE - 1) // PAGE) * PAGE if window else 0
        kp, vp, table = _paged([min(n, ring) if ring else n for n in lens], nkv, hd, 48, seed)
        q = (torch.randn(len(lens), nh * hd, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed))
             ).bfloat16()
        la = torch.tensor(lens, dtype=torch.int32, device="cuda")
        want = ops.attn_decode_tma(q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, splits)
        status, got = _call_noalloc(ops, lib, q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, splits)
        assert status == 0, lib.tb_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1e-2 * max(1.0, float(want.float().abs().max())), err     # the kernel tests' bfloat16 tolerance
        assert torch.equal(got, want)       # same kernel, same order of sums: in fact the same bits
    assert ops.attn_decode_error() == 0


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold():
    from trapetum_b200.csrc import build, ops
    lib = build.load("attention_decode")
    nh, nkv, hd, B, splits = 8, 4, 256, 64, 16          # 64 * 8 * 16 * 258 floats = 2.1M > 1M
    kp, vp, table = _paged([64] * B, nkv, hd, B, 3)
    q = torch.zeros(B, nh * hd, dtype=torch.bfloat16, device="cuda")
    la = torch.full((B,), 64, dtype=torch.int32, device="cuda")
    status, _ = _call_noalloc(ops, lib, q, kp, vp, table, la, nh, nkv, hd, 1.0, 0.0, 0, 0, splits)
    assert status < 0
    msg = lib.tb_error().decode()
    assert "2113536" in msg and "1048576" in msg
    status, out = _call_noalloc(ops, lib, q, kp, vp, table, la, nh, nkv, hd, 1.0, 0.0, 0, 0, 1)   # no splits: no scratch
    assert status == 0
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()

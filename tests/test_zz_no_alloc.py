"""The decode attention entry point that allocates nothing (attention_decode_noalloc.h), called the way
a C program would call it: a small C file, compiled by the test against the public header, fills the
argument block, looks the exported symbol up and calls it with a caller-owned output buffer.

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


_CALLER_C = r"""
/* A caller as a C program would write it: it includes the public header, fills the argument block
 * field by field, finds the exported symbol with dlsym and calls it. */
#include <dlfcn.h>
#include <string.h>
#include "attention_decode_noalloc.h"

typedef int (*noalloc_fn)(const DecodeArgs*, int, int, cudaStream_t);

unsigned long decode_args_bytes(void) { return sizeof(DecodeArgs); }

int call_noalloc(const char* library, const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                 const int* page_table, int pt_stride, const int* len_after, void* out, int n_heads, int n_kv_heads,
                 int hd, int ring_rows, int window, int n_splits, float scale, float cap, int dtype, int batch,
                 void* stream) {
    void* h = dlopen(library, RTLD_NOW | RTLD_LOCAL);
    if (!h) return -1000;
    noalloc_fn fn = (noalloc_fn)dlsym(h, "tb_attn_decode_noalloc");
    if (!fn) return -1001;
    DecodeArgs a;
    memset(&a, 0, sizeof a);
    a.q = q; a.q_stride = q_stride; a.k_pool = k_pool; a.v_pool = v_pool;
    a.page_table = page_table; a.pt_stride = pt_stride; a.len_after = len_after; a.out = out;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = hd; a.page_rows = 64;
    a.ring_rows = ring_rows; a.window = window; a.n_splits = n_splits; a.scale = scale; a.cap = cap;
    return fn(&a, dtype, batch, (cudaStream_t)stream);
}
"""


@pytest.fixture(scope="module")
def caller(tmp_path_factory):
    """The C caller above, compiled against the library's public header with the host compiler."""
    import os
    import subprocess
    from trapetum_b200.csrc import build
    d = tmp_path_factory.mktemp("noalloc_caller")
    src, out = os.path.join(d, "caller.c"), os.path.join(d, "caller.so")
    with open(src, "w") as f:
        f.write(_CALLER_C)
    csrc = os.path.dirname(os.path.abspath(build.__file__))
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(build._nvcc())), "include")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-I", csrc, "-I", cuda_inc, src, "-o", out, "-ldl"], check=True)
    lib = ctypes.CDLL(out)
    lib.decode_args_bytes.restype = ctypes.c_ulong
    lib.call_noalloc.restype = ctypes.c_int
    return lib


def _call_noalloc(caller, ops, q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, splits):
    """Call the exported C symbol through the C caller; the output buffer is the caller's."""
    from trapetum_b200.csrc import build
    out = torch.empty((q.shape[0], nh * hd), dtype=q.dtype, device=q.device)
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    status = caller.call_noalloc(build.library_path("attention_decode").encode(), P(q.data_ptr()), L(q.stride(0)),
                                 P(kp.data_ptr()), P(vp.data_ptr()), P(table.data_ptr()), I(table.stride(0)),
                                 P(la.data_ptr()), P(out.data_ptr()), I(nh), I(nkv), I(hd), I(ring), I(window), I(splits),
                                 F(scale), F(cap), I(ops.code(q.dtype)), I(q.shape[0]),
                                 P(torch.cuda.current_stream().cuda_stream))
    return status, out


def test_argument_block_is_the_same_in_c_and_in_python(caller):
    from trapetum_b200.csrc import ops
    assert caller.decode_args_bytes() == ctypes.sizeof(ops._DecodeArgs)


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(caller):
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
        status, got = _call_noalloc(caller, ops, q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, splits)
        assert status == 0, lib.tb_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1e-2 * max(1.0, float(want.float().abs().max())), err     # the kernel tests' bfloat16 tolerance
        assert torch.equal(got, want)       # same kernel, same order of sums: in fact the same bits
    assert ops.attn_decode_error() == 0


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold(caller):
    from trapetum_b200.csrc import build, ops
    lib = build.load("attention_decode")
    nh, nkv, hd, B, splits = 8, 4, 256, 64, 16          # 64 * 8 * 16 * 258 floats = 2.1M > 1M
    kp, vp, table = _paged([64] * B, nkv, hd, B, 3)
    q = torch.zeros(B, nh * hd, dtype=torch.bfloat16, device="cuda")
    la = torch.full((B,), 64, dtype=torch.int32, device="cuda")
    status, _ = _call_noalloc(caller, ops, q, kp, vp, table, la, nh, nkv, hd, 1.0, 0.0, 0, 0, splits)
    assert status < 0
    msg = lib.tb_error().decode()
    assert "2113536" in msg and "1048576" in msg
    status, out = _call_noalloc(caller, ops, q, kp, vp, table, la, nh, nkv, hd, 1.0, 0.0, 0, 0, 1)   # no splits: no scratch
    assert status == 0
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()

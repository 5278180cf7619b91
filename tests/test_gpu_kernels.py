"""Each CUDA kernel alone against a plain float32 torch formula, at sizes the engine's tiny
models do not use (odd widths, head sizes in steps of 16, group sizes, long rows)."""
import math

import pytest
import torch

import plain_gemma2 as plain

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]
PAGE = 64


@pytest.fixture(scope="module")
def ops():
    from trapetum_b200.csrc import ops as o
    assert torch.cuda.is_available(), "these tests need a GPU"
    return o


def tol(dt):
    return 2e-6 if dt == torch.float32 else 1e-2


def close(got, want, dt, scale=1.0):
    got, want = got.float().cpu(), want.float().cpu()
    err = float((got - want).abs().max())
    ref = float(want.abs().max()) + 1e-6
    assert err <= tol(dt) * scale * max(ref, 1.0), f"max abs err {err} (ref max {ref})"


def rnd(*shape, dt=torch.float32, s=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, device="cuda", generator=g) * s).to(dt)


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("V,H", [(50, 24), (301, 1000), (1024, 2304)])
def test_embed(ops, dt, V, H):
    table = rnd(V, H, dt=dt)
    ids = torch.tensor([0, V - 1, 3, 3, V // 2], dtype=torch.int32, device="cuda")
    out = ops.embed(ids, table, 7.5)
    assert out.dtype == torch.float32
    assert torch.equal(out, table.float()[ids.long()] * 7.5)
    bad = ops.embed(torch.tensor([V, -1], dtype=torch.int32, device="cuda"), table, 1.0)
    assert torch.isnan(bad).all()                     # an id outside the table cannot pass for a result


def test_gather_rows(ops):
    x = rnd(37, 131)
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.gather_rows(x, rows), x[rows.long()])


@pytest.mark.parametrize("xdt", DT)
@pytest.mark.parametrize("wdt", DT)
@pytest.mark.parametrize("odt", DT)
@pytest.mark.parametrize("rows,width,eps,off", [(3, 17, 1e-6, 1.0), (5, 2304, 1e-5, 1.0), (2, 5000, 1e-3, 0.0)])
def test_rmsnorm(ops, xdt, wdt, odt, rows, width, eps, off):
    x, w = rnd(rows, width, dt=xdt, s=3.0), rnd(width, dt=wdt, s=0.3)
    got = ops.rmsnorm(x, w, eps, off, odt)
    xf, wf = x.float(), w.float()
    want = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * (off + wf)
    close(got, want, odt)


@pytest.mark.parametrize("adt", DT)
@pytest.mark.parametrize("odt", DT)
@pytest.mark.parametrize("rows,width", [(4, 72), (3, 2304), (1, 4099)])
def test_add_rmsnorm(ops, adt, odt, rows, width):
    h0, a = rnd(rows, width, s=2.0), rnd(rows, width, dt=adt, s=5.0, seed=1)
    wa, wb = rnd(width, dt=odt, s=0.2, seed=2), rnd(width, dt=odt, s=0.2, seed=3)
    af = a.float()
    add = af * torch.rsqrt((af * af).mean(-1, keepdim=True) + 1e-6) * (1.0 + wa.float())
    h = h0.clone()
    assert ops.add_rmsnorm(h, a, wa, 1e-6, 1.0) is None
    close(h, h0 + add, torch.float32, 2.0)
    h = h0.clone()
    x = ops.add_rmsnorm(h, a, wa, 1e-6, 1.0, wb, 1e-5, 0.0, odt)
    hn = h0 + add
    close(h, hn, torch.float32, 2.0)
    close(x, hn * torch.rsqrt((hn * hn).mean(-1, keepdim=True) + 1e-5) * wb.float(), odt, 2.0)
    h = h0.clone()
    ops.residual_add(h, a)
    close(h, h0 + af, torch.float32)


@pytest.mark.parametrize("odt", DT)
@pytest.mark.parametrize("rows,width", [(64, 2304), (100, 3584), (65, 4608), (300, 520), (70, 72), (64, 5120)])
def test_add_rmsnorm_many_rows(ops, odt, rows, width):
    """Many rows take the warp-per-row kernel (32-bit branch, bfloat16 weights); same numbers as the formula."""
    h0, a = rnd(rows, width, s=2.0), rnd(rows, width, s=5.0, seed=1)
    wa, wb = rnd(width, dt=torch.bfloat16, s=0.2, seed=2), rnd(width, dt=torch.bfloat16, s=0.2, seed=3)
    add = a * torch.rsqrt((a * a).mean(-1, keepdim=True) + 1e-6) * (1.0 + wa.float())
    hn = h0 + add
    h = h0.clone()
    x = ops.add_rmsnorm(h, a, wa, 1e-6, 1.0, wb, 1e-5, 1.0, odt)
    close(h, hn, torch.float32, 2.0)
    close(x, hn * torch.rsqrt((hn * hn).mean(-1, keepdim=True) + 1e-5) * (1.0 + wb.float()), odt, 2.0)
    h = h0.clone()
    assert ops.add_rmsnorm(h, a, wa, 1e-6, 1.0) is None
    close(h, hn, torch.float32, 2.0)


@pytest.mark.parametrize("rows,width,splits", [(8, 2304, 8), (3, 72, 2), (1, 12000, 5)])
def test_add_rmsnorm_from_partial_sums(ops, rows, width, splits):
    part = rnd(splits, rows, width, s=2.0)
    h0 = rnd(rows, width, seed=5)
    wa, wb = rnd(width, dt=torch.bfloat16, s=0.2, seed=2), rnd(width, dt=torch.bfloat16, s=0.2, seed=3)
    a = part[0].clone()
    for s_ in range(1, splits):
        a += part[s_]                                                # the kernel adds in split order too
    h1, h2 = h0.clone(), h0.clone()
    x1 = ops.add_rmsnorm(h1, a, wa, 1e-6, 1.0, wb, 1e-6, 1.0, torch.bfloat16)
    x2 = ops.add_rmsnorm(h2, part, wa, 1e-6, 1.0, wb, 1e-6, 1.0, torch.bfloat16)
    assert torch.equal(h1, h2) and torch.equal(x1, x2)
    assert torch.equal(ops.sum_partials(part), a)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_gated_act(ops, dt, act):
    gu = rnd(5, 2 * 333, dt=dt, s=2.0)
    g, u = gu.float()[:, :333], gu.float()[:, 333:]
    want = (plain.gelu_tanh(g) if act == "gelu_tanh" else g * torch.sigmoid(g)) * u
    close(ops.gated_act(gu, act, dt), want, dt)


@pytest.mark.parametrize("adt,wdt,odt", [(torch.float32, torch.float32, torch.float32),
                                         (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                         (torch.bfloat16, torch.float32, torch.float32),
                                         (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (7, 301, 100), (65, 130, 77), (200, 64, 1030)])
def test_gemm_simt(ops, adt, wdt, odt, M, N, K):
    a, w = rnd(M, K, dt=adt, s=0.5), rnd(N, K, dt=wdt, s=0.5, seed=1)
    want = a.double() @ w.double().T
    close(ops.gemm_simt(a, w, odt), want, odt, scale=math.sqrt(K))
    close(ops.gemm_simt(a, w, torch.float32, softcap=3.0), 3.0 * torch.tanh(want / 3.0), torch.float32, scale=4.0)


def test_gemm_simt_row_does_not_depend_on_the_batch(ops):
    a, w = rnd(50, 333), rnd(97, 333, seed=1)
    full = ops.gemm_simt(a, w, torch.float32)
    one = ops.gemm_simt(a[17:18].contiguous(), w, torch.float32)
    assert torch.equal(full[17:18], one)


@pytest.mark.parametrize("odt", DT)
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (3, 40, 72), (16, 384, 96), (17, 130, 64), (64, 2304, 2048),
                                   (100, 512, 520), (128, 256, 64), (129, 256, 64), (300, 520, 200),
                                   (1000, 301 * 8, 1032), (2048, 1024, 2304), (2048, 10240, 128)])
@pytest.mark.parametrize("pair", [0, 1])
def test_gemm_tc(ops, odt, M, N, K, pair):
    """Few tokens (swapped tiles), many tokens on single SMs and on pairs of SMs (one tile a pair, and several)."""
    if pair and (M <= 128 or N < 256):
        pytest.skip("the pair kernel takes more than 128 tokens and at least 256 weight rows")
    a, w = rnd(M, K, dt=torch.bfloat16, s=0.5), rnd(N, K, dt=torch.bfloat16, s=0.5, seed=1)
    assert ops.gemm_tc_takes(a, w)
    want = a.double() @ w.double().T
    was = ops.gemm_tc_set_pair(pair)
    try:
        got = ops.gemm_tc(a, w, odt)
    finally:
        ops.gemm_tc_set_pair(was)
    torch.cuda.synchronize()
    assert ops.gemm_tc_error() == 0
    if odt == torch.float32:
        assert float((got.double() - want).norm() / want.norm()) < 2e-5
    else:
        assert float((got.double() - want).norm() / want.norm()) < 4e-3


@pytest.mark.parametrize("M,N,K,splits", [(8, 2304, 2048, 8), (64, 640, 9216, 5), (1, 136, 1024, 16), (33, 100 * 8, 520, 3)])
def test_gemm_tc_split_k(ops, M, N, K, splits):
    a, w = rnd(M, K, dt=torch.bfloat16, s=0.5), rnd(N, K, dt=torch.bfloat16, s=0.5, seed=1)
    want = a.double() @ w.double().T
    got = ops.gemm_tc(a, w, torch.float32, 0.0, splits)
    again = ops.gemm_tc(a, w, torch.float32, 0.0, splits)
    assert torch.equal(got, again)                                  # fixed summation order
    assert float((got.double() - want).norm() / want.norm()) < 2e-5
    capped = ops.gemm_tc(a, w, torch.float32, 5.0, splits)
    assert float((capped.double() - 5 * torch.tanh(want / 5)).abs().max()) < 1e-4
    assert ops.gemm_tc_error() == 0


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("M,I,K", [(1, 160, 96), (8, 9216, 2304), (40, 128, 64), (64, 1024, 512), (128, 176, 72),
                                   (129, 160, 96), (700, 1296, 520), (2048, 2048, 256)])
@pytest.mark.parametrize("pair", [0, 1])
def test_gemm_tc_gated_epilogue(ops, act, M, I, K, pair):
    """act(x Wg^T) * (x Wu^T) in the product's epilogue, swapped tiles (few tokens) and token-major ones, these on
    single SMs and on pairs."""
    if pair and M <= 128:
        pytest.skip("the pair kernel takes more than 128 tokens")
    x = rnd(M, K, dt=torch.bfloat16, s=1.0)
    wg, wu = rnd(I, K, dt=torch.bfloat16, s=0.1, seed=1), rnd(I, K, dt=torch.bfloat16, s=0.1, seed=2)
    g, u = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = (plain.gelu_tanh(g) if act == "gelu_tanh" else g * torch.sigmoid(g)) * u
    was = ops.gemm_tc_set_pair(pair)
    try:
        got = ops.gemm_tc(x, ops.interleave_gate_up(wg, wu), torch.bfloat16, gated_act=act)
    finally:
        ops.gemm_tc_set_pair(was)
    assert got.shape == (M, I) and got.dtype == torch.bfloat16
    assert float((got.double() - want).norm() / want.norm()) < 4e-3
    assert ops.gemm_tc_error() == 0


def test_gemm_tc_pair_policy_and_cap(ops):
    """The default policy sends a long product to pairs of SMs and a short one to single SMs; either way the result
    is the same up to the order of additions inside an instruction, with a soft cap and through a row-strided view."""
    big = rnd(2048, 2 * 4096, dt=torch.bfloat16, s=0.5)
    a = big[:, 4096:]                                                # row stride 8192
    w = rnd(16384 + 8, 4096, dt=torch.bfloat16, s=0.05, seed=1)      # 8 x 65 tiles of 64 k-blocks: long enough for the pair
    want = 5 * torch.tanh(a.double() @ w.double().T / 5)
    outs = []
    for mode in (0, 1, 2):
        was = ops.gemm_tc_set_pair(mode)
        try:
            outs.append(ops.gemm_tc(a, w, torch.float32, 5.0))
        finally:
            ops.gemm_tc_set_pair(was)
    assert was == 2                                                  # the default
    for got in outs:
        assert float((got.double() - want).abs().max()) < 1e-4
    assert torch.equal(outs[2], outs[1])                             # where the pair pays
    short = rnd(520, 64, dt=torch.bfloat16, s=0.5, seed=2)
    x = rnd(300, 64, dt=torch.bfloat16, s=0.5, seed=3)
    ops.gemm_tc_set_pair(0)
    try:
        single = ops.gemm_tc(x, short, torch.float32)
    finally:
        ops.gemm_tc_set_pair(2)
    assert torch.equal(ops.gemm_tc(x, short, torch.float32), single)  # a short product stays on single SMs
    assert ops.gemm_tc_error() == 0


def test_gemm_tc_views_and_refusals(ops):
    big = rnd(40, 3 * 256, dt=torch.bfloat16, s=0.5)
    w = rnd(96, 256, dt=torch.bfloat16, s=0.5, seed=1)
    a = big[:, 256:512]                                              # a column slice: row stride 768
    got = ops.gemm_tc(a, w, torch.float32)
    assert float((got.double() - a.double() @ w.double().T).abs().max()) < 1e-3
    assert not ops.gemm_tc_takes(rnd(4, 100, dt=torch.bfloat16), rnd(8, 100, dt=torch.bfloat16))   # K % 8
    assert not ops.gemm_tc_takes(rnd(4, 64), rnd(8, 64))                                         # float32
    with pytest.raises(ops.KernelError, match="does not take"):
        ops.gemm_tc(rnd(4, 100, dt=torch.bfloat16), rnd(8, 100, dt=torch.bfloat16), torch.float32)


def test_gemm_tc_token_rows_do_not_depend_on_the_batch(ops):
    """The same token row gives the same bits alone (swapped tiles) and among 40 rows."""
    a, w = rnd(40, 512, dt=torch.bfloat16, s=0.5), rnd(384, 512, dt=torch.bfloat16, s=0.5, seed=1)
    full = ops.gemm_tc(a, w, torch.float32, splits=1)
    one = ops.gemm_tc(a[7:8].contiguous(), w, torch.float32, splits=1)
    assert torch.equal(full[7:8], one)


# ---------------------------------------------------------------------------
def paged(k, v, lens, ring_rows, n_pages, seed=0):
    """Scatter dense per-sequence k, v ([len, nkv, hd] each) into scrambled pages; untouched rows are NaN."""
    nkv, hd = k[0].shape[1:]
    dt = k[0].dtype
    kp = torch.full((n_pages, nkv, PAGE, hd), float("nan"), dtype=dt, device="cuda")
    vp = torch.full((n_pages, nkv, PAGE, hd), float("nan"), dtype=dt, device="cuda")
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max((min(n, ring_rows) if ring_rows else n) + PAGE - 1 for n in lens) // PAGE
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    for b, n in enumerate(lens):
        rows = min(n, ring_rows) if ring_rows else n
        for pg in range((rows + PAGE - 1) // PAGE):
            table[b, pg] = perm.pop()
        for p in range(max(0, n - ring_rows) if ring_rows else 0, n):
            r = p % ring_rows if ring_rows else p
            page = int(table[b, r // PAGE])
            kp[page, :, r % PAGE, :] = k[b][p]
            vp[page, :, r % PAGE, :] = v[b][p]
    return kp, vp, table.cuda()


def ref_attention_one(q, k, v, scale, cap, window):
    """q [nh, hd] at position len-1 against k, v [len, nkv, hd] -> [nh, hd] (float64)."""
    n, nkv, hd = k.shape
    nh = q.shape[0]
    out = torch.zeros(nh, hd, dtype=torch.float64)
    lo = max(0, n - window) if window else 0
    for h in range(nh):
        kh = h // (nh // nkv)
        s = (k[lo:, kh].double() @ q[h].double()) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        p = torch.softmax(s, 0)
        out[h] = p @ v[lo:, kh].double()
    return out


def decode_impls(ops, dt, nh, nkv, hd):
    """The generic kernel always; the bulk-copy kernel too where it takes the shape."""
    import functools
    impls = [ops.attn_decode_simt]
    if ops.attn_decode_takes(dt, nh, nkv, hd):
        impls.append(ops.attn_decode_tma)
        if ops.attn_decode_stream_takes(dt, nh, nkv, hd, 64):
            # the stream partition, with CTA counts that leave parts of a sequence to several CTAs, one page to
            # each CTA (more CTAs than pages), and everything to one CTA; `splits` is not used by it
            for n_ctas in (None, 7, 1, 1000):
                def stream(q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, splits, n_ctas=n_ctas):
                    return ops.attn_decode_stream(q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, n_ctas)
                stream.__name__ = f"attn_decode_stream[{n_ctas}]"
                impls.append(stream)
        if nh // nkv in (1, 2, 4, 8):
            lanes = functools.partial(ops.attn_decode_tma, variant="lanes")
            lanes.__name__ = "attn_decode_lanes"
            impls.append(lanes)
    return impls


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("nh,nkv,hd,cap,window,splits", [
    (4, 2, 16, 50.0, 0, 1), (6, 1, 32, 0.0, 40, 3), (3, 3, 48, 20.0, 70, 2), (8, 4, 256, 50.0, 0, 4),
    (5, 5, 80, 0.0, 128, 7), (8, 2, 128, 30.0, 100, 1), (8, 1, 64, 10.0, 0, 2), (4, 4, 32, 0.0, 64, 5),
    (16, 2, 256, 50.0, 200, 3), (2, 1, 128, 0.0, 0, 9), (8, 8, 64, 0.0, 300, 1), (6, 2, 64, 25.0, 90, 2),
    (5, 1, 128, 0.0, 0, 3), (14, 2, 256, 50.0, 0, 2)])
def test_attn_decode(ops, dt, nh, nkv, hd, cap, window, splits):
    lens = [1, 37, 64, 65, 200, 333]
    ring = ((window + PAGE - 1) // PAGE) * PAGE if window else 0
    ks = [rnd(n, nkv, hd, dt=dt, seed=i).cpu() for i, n in enumerate(lens)]
    vs = [rnd(n, nkv, hd, dt=dt, seed=10 + i).cpu() for i, n in enumerate(lens)]
    q = rnd(len(lens), nh * hd, dt=dt, seed=99)
    kp, vp, table = paged([k.cuda() for k in ks], [v.cuda() for v in vs], lens, ring, 64, seed=hd)
    la = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = 0.37 / math.sqrt(hd)
    for impl in decode_impls(ops, dt, nh, nkv, hd):
        got = impl(q, kp, vp, table, la, nh, nkv, hd, scale, cap, window, ring, splits)
        assert torch.isfinite(got.float()).all(), f"{impl.__name__}: a row outside the sequence's own keys was read"
        for b, n in enumerate(lens):
            want = ref_attention_one(q[b].view(nh, hd).cpu(), ks[b], vs[b], scale, cap, window)
            close(got[b].view(nh, hd), want, dt, 2.0)
    torch.cuda.synchronize()
    assert ops.attn_decode_error() == 0


@pytest.mark.parametrize("splits", [17, 33, 64, 70])
def test_attn_decode_in_many_pieces(ops, splits):
    """A long sequence cut into many pieces: the fold inside the kernel takes up to 32 pieces at a time and holds
    the weights of 64; more than 64 pieces go to the fold launch."""
    dt, nh, nkv, hd = torch.bfloat16, 4, 2, 64
    lens = [PAGE * 70 + 5, 300]
    ks = [rnd(n, nkv, hd, dt=dt, seed=i).cpu() for i, n in enumerate(lens)]
    vs = [rnd(n, nkv, hd, dt=dt, seed=10 + i).cpu() for i, n in enumerate(lens)]
    q = rnd(len(lens), nh * hd, dt=dt, seed=99)
    kp, vp, table = paged([k.cuda() for k in ks], [v.cuda() for v in vs], lens, 0, 80, seed=3)
    la = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = 0.37 / math.sqrt(hd)
    for rep in range(2):                                                # twice: the tickets are used again
        got = ops.attn_decode_tma(q, kp, vp, table, la, nh, nkv, hd, scale, 30.0, 0, 0, splits)
        assert torch.isfinite(got.float()).all()
        for b, n in enumerate(lens):
            want = ref_attention_one(q[b].view(nh, hd).cpu(), ks[b], vs[b], scale, 30.0, 0)
            close(got[b].view(nh, hd), want, dt, 2.0)
    torch.cuda.synchronize()
    assert ops.attn_decode_error() == 0


@pytest.mark.parametrize("nh,nkv,hd,rot,cap,window", [(8, 4, 256, 256, 50.0, 0), (8, 4, 256, 256, 50.0, 128), (6, 2, 64, 32, 0.0, 70),
                                                     (5, 5, 128, 0, 0.0, 0), (14, 2, 256, 64, 30.0, 200), (4, 1, 128, 128, 0.0, 64)])
def test_attn_decode_that_rotates_and_appends_by_itself(ops, nh, nkv, hd, rot, cap, window):
    """Given the partial sums of the q/k/v product, the tensor-core decode kernel must do what the rotation kernel
    followed by the attention kernel does: the same output, and the same new rows in the cache, bit for bit (same
    sums in the same order).  The new token lies on a page's first row, last row and in the middle; in a ring it
    overwrites the oldest row."""
    dt = torch.bfloat16
    lens = [1, 64, 65, 200, 333, 128]
    ring = ((window + PAGE - 1) // PAGE) * PAGE if window else 0
    ks = [rnd(n, nkv, hd, dt=dt, seed=i).cpu() for i, n in enumerate(lens)]
    vs = [rnd(n, nkv, hd, dt=dt, seed=10 + i).cpu() for i, n in enumerate(lens)]
    kp, vp, table = paged([k.cuda() for k in ks], [v.cuda() for v in vs], lens, ring, 64, seed=hd)
    la = torch.tensor(lens, dtype=torch.int32, device="cuda")
    B, width = len(lens), (nh + 2 * nkv) * hd
    part = rnd(3, B, width, dt=torch.float32, s=0.6, seed=5)         # three splits of the product
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).cuda() if rot else None
    pos = (la - 1).contiguous()
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    scale = 0.37 / math.sqrt(hd)
    # the two-kernel path, on its own copy of the cache
    kp1, vp1 = kp.clone(), vp.clone()
    qkv = torch.empty(B, width, dtype=dt, device="cuda")
    ops.rope_kv(qkv, nh, nkv, hd, rot, inv_freq, pos, seq, la, kp1, vp1, table, ring, part)
    want = ops.attn_decode_tma(qkv[:, :nh * hd], kp1, vp1, table, la, nh, nkv, hd, scale, cap, window, ring, 2)
    runs = [("split 1", lambda k, v: ops.attn_decode_tma(part, k, v, table, la, nh, nkv, hd, scale, cap, window, ring, 1, "mma", (inv_freq, rot))),
            ("split 3", lambda k, v: ops.attn_decode_tma(part, k, v, table, la, nh, nkv, hd, scale, cap, window, ring, 3, "mma", (inv_freq, rot)))]
    for n_ctas in (None, 5, 1, 1000):
        runs.append((f"stream {n_ctas}", lambda k, v, n_ctas=n_ctas: ops.attn_decode_stream(
            part, k, v, table, la, nh, nkv, hd, scale, cap, window, ring, n_ctas, (inv_freq, rot))))
    for name, run in runs:
        kp2, vp2 = kp.clone(), vp.clone()
        got = run(kp2, vp2)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all(), name
        # NaN marks rows that no token has written: equal_nan compares them too
        assert torch.equal(torch.nan_to_num(kp2.float(), nan=-7.0), torch.nan_to_num(kp1.float(), nan=-7.0)), f"{name}: k rows"
        assert torch.equal(torch.nan_to_num(vp2.float(), nan=-7.0), torch.nan_to_num(vp1.float(), nan=-7.0)), f"{name}: v rows"
        close(got, want, dt, 2.0)
    assert ops.attn_decode_error() == 0


@pytest.mark.parametrize("dt", DT)
def test_attn_decode_far_key_and_window_edge(ops, dt):
    """One key is made to stand out.  Among hundreds it must win the softmax; one step outside the
    window it must be invisible; on the window's first row it must be seen."""
    nh, nkv, hd, n, W = 2, 1, 32, 500, 128
    ring = 128
    for marked, sees in ((3, "full only"), (n - W - 1, "full only"), (n - W, "both"), (n - 1, "both")):
        k = rnd(n, nkv, hd, dt=dt, s=0.1, seed=marked)
        v = rnd(n, nkv, hd, dt=dt, s=1.0, seed=marked + 1)
        q = rnd(1, nh * hd, dt=dt, s=0.1, seed=7)
        k[marked, 0] = (q.view(nh, hd)[0].float() * 400).to(dt)        # q0 . k_marked is huge
        la = torch.tensor([n], dtype=torch.int32, device="cuda")
        for window, rr in ((0, 0), (W, ring)):
            kp, vp, table = paged([k], [v], [n], rr, 16, seed=1)
            for impl in decode_impls(ops, dt, nh, nkv, hd):
                got = impl(q, kp, vp, table, la, nh, nkv, hd, 1.0, 0.0, window, rr, 3).view(nh, hd)
                visible = window == 0 or sees == "both"
                hit = float((got[0].float() - v[marked, 0].float()).abs().max()) < 2e-2
                assert hit == visible, f"{impl.__name__}: key {marked}, window {window}: expected visible={visible}"


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("nh,nkv,hd,cap,window", [(4, 2, 16, 50.0, 8), (6, 1, 32, 0.0, 16), (3, 3, 48, 20.0, 0),
                                                  (2, 1, 256, 50.0, 50), (4, 4, 112, 0.0, 0), (4, 2, 64, 0.0, 64),
                                                  (2, 2, 128, 30.0, 65), (8, 4, 256, 50.0, 0)])
def test_attn_prefill(ops, dt, nh, nkv, hd, cap, window):
    lens = [1, 70, 9, 33, 200, 64, 129]
    T = sum(lens)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dt=dt, s=0.7)
    q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    seq_start = torch.tensor(starts, dtype=torch.int32, device="cuda")
    token_seq = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int32), torch.tensor(lens)).cuda()
    scale = 1.0 / math.sqrt(hd)
    impls = [lambda: ops.attn_prefill_simt(q, k, v, seq_start, token_seq, nh, nkv, hd, scale, cap, window)]
    if ops.attn_prefill_takes(dt, hd) and hd in (16, 32, 48, 64, 128, 256):
        impls.append(lambda: ops.attn_prefill_mma(q, k, v, seq_start, nh, nkv, hd, scale, cap, window, max(lens)))
    if ops.attn_prefill_tc_takes(dt, hd):
        impls.append(lambda: ops.attn_prefill_tc(q, k, v, seq_start, lens, nh, nkv, hd, scale, cap, window))
    wants = []
    for b, n in enumerate(lens):
        s = slice(starts[b], starts[b + 1])
        wants.append(plain.attention(q[s].float().cpu().view(n, nh, hd), k[s].float().cpu().view(n, nkv, hd),
                                     v[s].float().cpu().view(n, nkv, hd), scale, cap or None, window or None))
    for impl in impls:
        got = impl()
        for b, n in enumerate(lens):
            close(got[starts[b]:starts[b + 1]].view(n, nh, hd), wants[b], dt, 2.0)
    if ops.attn_prefill_tc_takes(dt, hd):
        torch.cuda.synchronize()
        assert ops.attn_prefill_tc_error(hd) == 0


@pytest.mark.parametrize("nh,nkv,hd,cap,window,lens", [(8, 4, 256, 50.0, 0, [1000]), (8, 4, 256, 50.0, 300, [700, 64, 129]),
                                                       (4, 1, 128, 0.0, 0, [513, 1]), (2, 2, 64, 20.0, 100, [400, 333]),
                                                       (4, 2, 256, 50.0, 1024, [2500]), (4, 2, 128, 30.0, 0, [2100, 700])])
def test_attn_prefill_tc_long(ops, nh, nkv, hd, cap, window, lens):
    """Long sequences: many key blocks, the lazy rescaling of O, the window's trailing edge, and query
    tiles whose rows belong to the next sequence of the packed batch."""
    T = sum(lens)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dt=torch.bfloat16, s=1.0)
    # make the scores grow along each sequence, so that the running maximum keeps moving
    ramp = torch.cat([torch.linspace(0.2, 2.0, n) for n in lens]).cuda().bfloat16()
    qkv[:, nh * hd:(nh + nkv) * hd] *= ramp[:, None]
    q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    seq_start = torch.tensor(starts, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    got = ops.attn_prefill_tc(q, k, v, seq_start, lens, nh, nkv, hd, scale, cap, window)
    ref = ops.attn_prefill_mma(q, k, v, seq_start, nh, nkv, hd, scale, cap, window, max(lens))
    torch.cuda.synchronize()
    assert ops.attn_prefill_tc_error(hd) == 0
    assert torch.isfinite(got.float()).all()
    for b, n in enumerate(lens):
        s = slice(starts[b], starts[b + 1])
        sub = slice(0, n) if n <= 400 else slice(n - 200, n)
        want = plain.attention(q[s].float().cpu().view(n, nh, hd), k[s].float().cpu().view(n, nkv, hd),
                               v[s].float().cpu().view(n, nkv, hd), scale, cap or None, window or None)
        close(got[s].view(n, nh, hd)[sub], want[sub], torch.bfloat16, 2.0)
        close(ref[s].view(n, nh, hd)[sub], want[sub], torch.bfloat16, 2.0)


def test_attn_prefill_far_key_and_window_edge(ops):
    """A key made to stand out is seen from far away without a window, and exactly up to the window's
    edge with one; on tensor cores and on the generic kernel alike."""
    nh, nkv, hd, n, W = 2, 1, 64, 300, 100
    qkv = rnd(n, (nh + 2 * nkv) * hd, dt=torch.bfloat16, s=0.1)
    q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
    marked = 37
    k[marked] = (q[250, :hd].float() * 300).to(torch.bfloat16)          # query 250, head 0 loves key 37
    for i in (marked + W - 1, marked + W, 250):
        q[i, :hd] = q[250, :hd]
    seq_start = torch.tensor([0, n], dtype=torch.int32, device="cuda")
    token_seq = torch.zeros(n, dtype=torch.int32, device="cuda")
    for window in (0, W):
        for got in (ops.attn_prefill_simt(q, k, v, seq_start, token_seq, nh, nkv, hd, 1.0, 0.0, window),
                    ops.attn_prefill_mma(q, k, v, seq_start, nh, nkv, hd, 1.0, 0.0, window, n),
                    ops.attn_prefill_tc(q, k, v, seq_start, [n], nh, nkv, hd, 1.0, 0.0, window)):
            got = got.view(n, nh, hd).float()
            hit = lambda i: float((got[i, 0] - v[marked].float()).abs().max()) < 3e-2
            assert hit(marked + W - 1)                                  # the window's last row that still sees it
            assert hit(marked + W) == (window == 0)                     # one further: only without a window
            assert hit(250) == (window == 0)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("hd,rot,ring,theta", [(16, 16, 0, 1e4), (48, 48, 128, 5e4), (256, 256, 64, 1e4), (32, 16, 0, 1e3), (64, 0, 0, 1.0),
                                               (640, 640, 0, 1e4), (576, 530, 64, 1e4)])     # more pairs than a CTA has threads for
def test_rope_kv(ops, dt, hd, rot, ring, theta):
    nh, nkv = 3, 2
    lens_before, new = [0, 0, 0], [5, 150, 70]                      # a first step
    for lens_before, new in (([0, 0, 0], [5, 150, 70]), ([5, 150, 70], [1, 1, 1])):
        B, T = len(new), sum(new)
        qkv = rnd(T, (nh + 2 * nkv) * hd, dt=dt, seed=T)
        orig = qkv.clone()
        pos = torch.cat([torch.arange(b, b + n) for b, n in zip(lens_before, new)]).int().cuda()
        tseq = torch.repeat_interleave(torch.arange(B), torch.tensor(new)).int().cuda()
        after = [b + n for b, n in zip(lens_before, new)]
        la = torch.tensor(after, dtype=torch.int32, device="cuda")
        n_pages = 16
        kp = torch.full((n_pages, nkv, PAGE, hd), float("nan"), dtype=dt, device="cuda")
        vp = torch.full_like(kp, float("nan"))
        width = max(((min(a, ring) if ring else a) + PAGE - 1) // PAGE for a in after)
        table = torch.zeros(B, width, dtype=torch.int32)
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).tolist()
        for b, a in enumerate(after):
            for pg in range(((min(a, ring) if ring else a) + PAGE - 1) // PAGE):
                table[b, pg] = perm.pop()
        table = table.cuda()
        inv = (1.0 / (torch.tensor(theta) ** (torch.arange(0, rot, 2).float() / rot))).cuda() if rot else None
        if dt == torch.bfloat16 and T <= 16:
            # the same values as three partial sums: the kernel adds them, rotates in 32-bit, rounds once
            part = torch.stack([orig.float() * 0.5, orig.float() * 0.25, orig.float() * 0.25])
            dst = torch.full_like(qkv, float("nan"))
            kp2, vp2 = kp.clone(), vp.clone()
            ops.rope_kv(dst, nh, nkv, hd, rot, inv, pos, tseq, la, kp2, vp2, table, ring, partial=part)
        ops.rope_kv(qkv, nh, nkv, hd, rot, inv, pos, tseq, la, kp, vp, table, ring)
        if dt == torch.bfloat16 and T <= 16:
            assert torch.equal(dst, qkv) and torch.equal(torch.nan_to_num(kp2.float()), torch.nan_to_num(kp.float())) \
                and torch.equal(torch.nan_to_num(vp2.float()), torch.nan_to_num(vp.float()))
        o = orig.float().cpu().view(T, nh + 2 * nkv, hd)
        want = o.clone()
        if rot:
            want[:, :nh + nkv, :rot] = plain.rope(o[:, :nh + nkv, :rot], pos.cpu(), theta)
        got = qkv.float().cpu().view(T, nh + 2 * nkv, hd)
        close(got, want, dt, 2.0)
        assert torch.equal(got[:, nh + nkv:], o[:, nh + nkv:])       # v is not rotated
        # every token that must be in the cache is there, at its row, and nothing else was written
        written = 0
        for t in range(T):
            b, p = int(tseq[t]), int(pos[t])
            if ring and p < after[b] - ring:
                continue
            r = p % ring if ring else p
            page = int(table[b, r // PAGE])
            assert torch.equal(kp[page, :, r % PAGE].float().cpu(), got[t, nh:nh + nkv])
            assert torch.equal(vp[page, :, r % PAGE].float().cpu(), got[t, nh + nkv:])
            written += 1
        assert int((~torch.isnan(kp.float()[:, 0, :, 0])).sum()) == written


# ---------------------------------------------------------------------------
def test_argmax_ties_and_rows(ops):
    V = 256000
    x = rnd(5, V)
    x[0, 1234] = x[0, 200000] = 50.0            # a tie: the smaller index wins
    x[1, V - 1] = 60.0
    x[2, 0] = 60.0
    x[3, :] = -1.0                              # all equal
    x[4, 8191] = x[4, 8192] = 70.0              # a tie across the border of two stage-one chunks
    got = ops.argmax(x).cpu().tolist()
    assert got == [1234, V - 1, 0, 0, 8191]
    assert ops.argmax(rnd(3, 301)).cpu().tolist() == rnd(3, 301).argmax(-1).cpu().tolist()


def _args(rows, temperature, top_p, penalty, draws):
    f = lambda v: torch.full((rows,), float(v), device="cuda") if not isinstance(v, torch.Tensor) else v.cuda().float()
    return f(temperature), f(top_p), f(penalty), f(draws)


@pytest.mark.parametrize("V", [1000, 40001])      # one CTA a row; several CTAs a row (the ids lie in different chunks)
def test_sample_greedy_and_penalty(ops, V):
    a, b, c, d = 10, V - 7, V // 2 + 3, 5
    x = rnd(4, V)
    x[:, a] = 9.0; x[:, b] = 8.0
    recent = torch.full((4, 128), -1, dtype=torch.int32, device="cuda")
    recent[1, :3] = torch.tensor([a, a, d], dtype=torch.int32)          # a twice: penalised once
    recent[1, 100] = a
    recent[2, 0] = b
    x[3, a] = -0.5; x[3, b] = -0.6; x[3, c] = -0.55
    x[3, :] = torch.minimum(x[3, :], torch.tensor(-0.5, device="cuda"))
    recent[3, 0] = a
    before = x.clone()
    t, p, pen, u = _args(4, 0.0, 0.95, 1.2, 0.5)
    got = ops.sample(x, t, p, pen, u, recent).cpu().tolist()
    want = [plain.greedy(plain.repetition_penalty(before[i].cpu(), recent[i].cpu().tolist(), 1.2)) for i in range(4)]
    assert got == want and got[0] == a and got[1] == b and got[2] == a
    assert float(x[1, a]) == pytest.approx(9.0 / 1.2) and float(x[1, d]) == pytest.approx(
        float(before[1, d]) / 1.2 if before[1, d] > 0 else float(before[1, d]) * 1.2)


@pytest.mark.parametrize("V", [301, 256000])
@pytest.mark.parametrize("temperature,top_p", [(1.0, 1.0), (0.7, 0.95), (1.5, 0.5), (0.3, 0.9)])
def test_sample_draws_follow_the_inverse_cdf(ops, V, temperature, top_p):
    rows = 32
    x = rnd(rows, V, s=2.0, seed=V)
    u = torch.linspace(0.001, 0.999, rows)
    t, p, pen, ud = _args(rows, temperature, top_p, 1.0, u)
    got = ops.sample(x.clone(), t, p, pen, ud, None).cpu().tolist()
    for i in range(rows):
        probs = plain.nucleus(x[i].cpu(), temperature, top_p)          # float64, renormalised over the nucleus
        cdf = torch.cumsum(probs, 0)
        tok = got[i]
        assert probs[tok] > 0, "a token outside the nucleus was drawn"
        lo = float(cdf[tok] - probs[tok])
        assert lo - 1e-4 <= float(u[i]) <= float(cdf[tok]) + 1e-4


@pytest.mark.parametrize("V", [500, 20011])
def test_sample_mixed_rows(ops, V):
    x = rnd(3, V, s=3.0)
    t = torch.tensor([0.0, 1.0, 0.0]); p = torch.tensor([1.0, 1.0, 1.0])
    got = ops.sample(x.clone(), t.cuda(), p.cuda(), torch.ones(3).cuda(), torch.tensor([0.3, 0.3, 0.3]).cuda(), None)
    assert got[0] == x[0].argmax() and got[2] == x[2].argmax()


def test_refusals(ops):
    with pytest.raises(ops.KernelError, match="GPU only"):
        ops.rmsnorm(torch.zeros(2, 4), torch.zeros(4), 1e-6, 1.0, torch.float32)
    with pytest.raises(ops.KernelError, match="heads"):
        ops.attn_prefill_simt(rnd(2, 48), rnd(2, 32), rnd(2, 32), torch.zeros(2, dtype=torch.int32, device="cuda"),
                              torch.zeros(2, dtype=torch.int32, device="cuda"), 3, 2, 16, 1.0, 0.0, 0)
    with pytest.raises(ops.KernelError, match="512"):
        ops.attn_prefill_simt(rnd(2, 1024), rnd(2, 1024), rnd(2, 1024), torch.zeros(2, dtype=torch.int32, device="cuda"),
                              torch.zeros(2, dtype=torch.int32, device="cuda"), 1, 1, 1024, 1.0, 0.0, 0)
    with pytest.raises(ops.KernelError, match="float32 and bfloat16"):
        ops.rmsnorm(torch.zeros(2, 4, device="cuda", dtype=torch.float16), torch.zeros(4, device="cuda"), 1e-6, 1.0,
                    torch.float32)


def test_attn_decode_ctas_per_sm(ops):
    """The tensor-core decode kernel's stream partition is budgeted (shared memory to the byte, registers by its
    launch bounds) for two CTAs an SM at heads narrower than 256: if a change breaks the budget the kernel still
    computes the same, only slower, so the fit is checked here."""
    from trapetum_b200.csrc import build
    lib = build.load("attention_decode")
    for hd in (64, 128, 256):
        assert lib.tb_attn_decode_occupancy(hd, 0) == 1, hd
        assert lib.tb_attn_decode_occupancy(hd, 1) == (2 if hd <= 128 else 1), hd

"""The engine against the plain implementation, in float32 and in bfloat16: every way of cutting
the same requests into steps and batches must give the same logits."""
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_gemma2 as plain
from conftest import ROOT, TINY, TOL, bf16_budget, make_prompts, rel_l2, within

pytestmark = pytest.mark.gpu

NAMES = ["A", "B", "C"]
DTYPES = ["float32", "bfloat16"]
HOSTS = ["native", "python"]          # the C++ host (the default for these models) and the Python host
TOLERANCE = {}       # "of": (model name, token ids, dtype) -> tolerance, set from the fixture below


@pytest.fixture(scope="module")
def engines(model_folders):
    import trapetum_b200 as tb
    cache = {}

    def get(name, dtype, max_tokens=64 * 40, host=None):
        key = (name, dtype, max_tokens, host)
        if key not in cache:
            model = tb.load_model(model_folders[name], dtype, host=host)
            eng = tb.Engine(model, max_tokens=max_tokens)
            for g in eng.cache.groups:                      # a row that was never written reads as NaN
                g.k.fill_(float("nan")); g.v.fill_(float("nan"))
            cache[key] = eng
        return cache[key]
    return get


@pytest.fixture(scope="module", autouse=True)
def _tolerances(tolerance_of):
    TOLERANCE["of"] = tolerance_of


@pytest.fixture(scope="module")
def requests_and_truth(plain_models):
    """Per config: prompts of unequal lengths (longer than the windows and than one page) and the
    plain implementation's logits for every position."""
    out = {}
    for name in NAMES:
        cfg, w = plain_models[name]
        prompts = make_prompts(cfg["vocab_size"], [45, 77, 150, 33, 101, 64], seed=11 + len(name))
        out[name] = (prompts, [plain.forward(cfg, w, p) for p in prompts])
    return out


def check(got, want, dtype, what, ids):
    """``ids``: the sequence whose logits these are; its tolerance comes from the oracle for this sequence."""
    assert got.shape == want.shape, what
    assert torch.isfinite(got).all(), f"{what}: NaN or inf in the logits"
    worst = max(rel_l2(got[i], want[i]) for i in range(got.shape[0]))
    within(worst, TOLERANCE["of"](what.split()[0], ids, dtype), dtype, what)
    if dtype == "float32":
        assert (got.cpu().argmax(-1) == want.argmax(-1)).all(), f"{what}: top-1 differs"


@pytest.mark.parametrize("host", HOSTS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(engines, requests_and_truth, name, dtype, host):
    eng = engines(name, dtype, host=host)
    prompts, truth = requests_and_truth[name]
    for p, t in zip(prompts, truth):
        s = eng.start(1)
        got = eng.step(s, [p], [list(range(len(p)))])
        eng.release(s)
        check(got, t, dtype, f"{name} whole, {len(p)} tokens", p)
    eng.cache.check()
    assert eng.cache.live_slots() == []


@pytest.mark.parametrize("host", HOSTS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(engines, requests_and_truth, name, dtype, host):
    eng = engines(name, dtype, host=host)
    prompts, truth = requests_and_truth[name]
    for p, t in zip(prompts, truth):
        n = len(p) - 32
        s = eng.start(1)
        got = [eng.step(s, [p[:n]], [list(range(n))])]
        for i in range(n, len(p)):
            got.append(eng.step(s, [[p[i]]], [[0]]))
        eng.release(s)
        check(torch.cat(got), t, dtype, f"{name} tail one by one, {len(p)} tokens", p)


@pytest.mark.parametrize("host", HOSTS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(engines, requests_and_truth, name, dtype, host):
    """Batches of unequal prompts; each request's prompt is its first part, the rest is fed one token
    per step; shorter requests end earlier and give their slot back while the others go on; the next
    batch starts in the slots (and pages) the first one used."""
    eng = engines(name, dtype, host=host)
    prompts, truth = requests_and_truth[name]
    cut = [20, 70, 9, 1, 66, 64]                 # prompt part of each request
    used_slots = []
    for batch in ([0, 1, 2], [3, 4, 5], [2, 0], [5]):
        slots = eng.start(len(batch))
        used_slots.append(list(slots))
        got = {r: [] for r in batch}
        first = eng.step(slots, [prompts[r][:cut[r]] for r in batch], [list(range(cut[r])) for r in batch])
        o = 0
        for r in batch:
            got[r].append(first[o:o + cut[r]]); o += cut[r]
        live = list(zip(batch, slots))
        t = 0
        while live:
            done = [(r, s) for r, s in live if cut[r] + t >= len(prompts[r])]
            for r, s in done:
                eng.release([s])
            live = [x for x in live if x not in done]
            if not live:
                break
            out = eng.step([s for _, s in live], [[prompts[r][cut[r] + t]] for r, _ in live])
            for i, (r, _) in enumerate(live):
                got[r].append(out[i:i + 1])
            t += 1
        for r in batch:
            check(torch.cat(got[r]), truth[r], dtype, f"{name} batch {batch}, request {r}", prompts[r])
        eng.cache.check()
    assert used_slots[1] == used_slots[0] and eng.cache.live_slots() == []     # slots were used again


@pytest.mark.parametrize("host", HOSTS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_and_first_tokens(engines, plain_models, name, dtype, host):
    """From a one-token prompt, 280 tokens one by one: across page borders, past the window, around
    the ring more than once.  The first positions of a sequence are checked on the way."""
    eng = engines(name, dtype, host=host)
    cfg, w = plain_models[name]
    ids = make_prompts(cfg["vocab_size"], [281], seed=5)[0]
    truth = plain.forward(cfg, w, ids)
    s = eng.start(1)
    got = [eng.step(s, [ids[:1]], [[0]])]
    for i in range(1, len(ids)):
        got.append(eng.step(s, [[ids[i]]]))
    eng.release(s)
    got = torch.cat(got)
    check(got[:4], truth[:4], dtype, f"{name} first tokens", ids)
    check(got, truth, dtype, f"{name} long decoding", ids)


@pytest.mark.parametrize("host", HOSTS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_second_batch_with_the_same_slots_and_page_counts_but_other_pages(model_folders, plain_models, name, dtype, host):
    """Batch one: two prompts of 40 tokens that decode 30 more, so each sequence ends with two pages, taken
    alternately ([0, 2] and [1, 3]).  Batch two, in the same slots: two prompts of 70 tokens, two pages each
    again, but taken in a row ([0, 1] and [2, 3]).  Its first decode step has the batch size, the length bucket
    and the page counts of batch one's last step; page tables kept from batch one would make sequence 0 read
    and write sequence 1's page."""
    import trapetum_b200 as tb
    cfg, w = plain_models[name]
    eng = tb.Engine(tb.load_model(model_folders[name], dtype, host=host), max_tokens=64 * 8)
    for g in eng.cache.groups:
        g.k.fill_(float("nan")); g.v.fill_(float("nan"))
    first = make_prompts(cfg["vocab_size"], [70, 70], seed=41)
    second = make_prompts(cfg["vocab_size"], [90, 90], seed=42)
    pages = []
    for reqs, cut in ((first, 40), (second, 70)):
        truth = [plain.forward(cfg, w, p) for p in reqs]
        slots = eng.start(2)
        got = [[x] for x in eng.step(slots, [p[:cut] for p in reqs], [list(range(cut))] * 2).split(cut)]
        for t in range(cut, len(reqs[0])):
            out = eng.step(slots, [[p[t]] for p in reqs])
            for i in range(2):
                got[i].append(out[i:i + 1])
            if t == cut:
                pages.append([[list(eng.cache.pages(s, gi)) for gi in range(len(eng.cache.groups))] for s in slots])
        pages.append([[len(eng.cache.pages(s, gi)) for gi in range(len(eng.cache.groups))] for s in slots])
        eng.release(slots)
        for i in range(2):
            check(torch.cat(got[i]), truth[i], dtype, f"{name} batch with {cut}-token prompts, request {i}", reqs[i])
    assert pages[1] == [[len(p) for p in seq] for seq in pages[2]]      # the counts repeat ...
    assert any(len(g) > 1 for seq in pages[2] for g in seq)             # ... over more than one page ...
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unsharpened_models_keep_the_flat_tolerance(tmp_path, name, dtype):
    """The same configurations with the weights as the generator makes them (no scaled q and k projections):
    here 16-bit storage costs little, and the bfloat16 engine has to stay within the flat 2e-2."""
    import trapetum_b200 as tb
    cfg, seed, std, nstd, _ = TINY[name]
    d = str(tmp_path / "plainweights")
    tb.write_random_model(d, cfg, seed + 50, std, nstd)
    pc, pw = plain.load_folder(d)
    prompts = make_prompts(cfg["vocab_size"], [90, 33], seed=8)
    truth = [plain.forward(pc, pw, p) for p in prompts]
    eng = tb.Engine(tb.load_model(d, dtype), max_tokens=64 * 4)
    cut = [60, 20]
    s = eng.start(2)
    first = eng.step(s, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut])
    worst = max(rel_l2(first[i], truth[0][i]) for i in range(cut[0]))
    worst = max(worst, max(rel_l2(first[cut[0] + i], truth[1][i]) for i in range(cut[1])))
    for t in range(13):
        out = eng.step(s, [[p[c + t]] for p, c in zip(prompts, cut)])
        worst = max(worst, rel_l2(out[0], truth[0][cut[0] + t]), rel_l2(out[1], truth[1][cut[1] + t]))
    eng.release(s)
    within(worst, TOL[dtype], dtype, f"{name} unsharpened")


def test_float16_checkpoint_is_kept_exactly(model_folders, plain_models, tmp_path):
    """The same weights stored in float16 (values that bfloat16 cannot hold: a multiple of 2^-10 is added):
    the bfloat16 engine widens them rather than rounding them, so its logits follow the float16 values."""
    import shutil
    import trapetum_b200 as tb
    from safetensors.torch import load_file, save_file
    d = str(tmp_path / "f16")
    shutil.copytree(model_folders["A"], d)
    w = load_file(d + "/model.safetensors")
    g = torch.Generator().manual_seed(0)
    w16 = {k: (v.float() * (1.0 + 2.0 ** -9 * torch.randint(0, 2, v.shape, generator=g))).to(torch.float16) for k, v in w.items()}
    save_file(w16, d + "/model.safetensors")
    cfg, pw = plain.load_folder(d)
    ids = make_prompts(cfg["vocab_size"], [50], seed=77)[0]
    truth = plain.forward(cfg, pw, ids)
    rounded = plain.forward(cfg, {k: v.bfloat16().float() for k, v in pw.items()}, ids)
    gap = max(rel_l2(rounded[i], truth[i]) for i in range(50))           # what silent rounding of the weights would cost
    for fp16, dtype in (("widen", "bfloat16"), ("widen", "float32")):
        model = tb.load_model(d, dtype, fp16=fp16)
        if hasattr(model, "blocks"):              # the Python host's model shows its bound weights
            assert model.blocks[0].mixer.w_qkv.dtype == torch.float32 and model.blocks[0].mixer.w_o.dtype == torch.float32
        eng = tb.Engine(model, max_tokens=128)
        s = eng.start(1)
        got = eng.step(s, [ids], [list(range(50))])
        eng.release(s)
        worst = max(rel_l2(got[i], truth[i]) for i in range(50))
        if dtype == "float32":
            assert worst < 1e-5 < gap
        else:
            within(worst, bf16_budget(cfg, pw, [ids]), dtype, "A stored in float16")


@pytest.mark.parametrize("name", NAMES)
def test_runs_repeat_bit_for_bit(engines, requests_and_truth, name):
    eng = engines(name, "bfloat16")
    prompts, _ = requests_and_truth[name]
    outs = []
    for _ in range(2):
        s = eng.start(2)
        a = eng.step(s, [prompts[0], prompts[1]], [[len(prompts[0]) - 1], [len(prompts[1]) - 1]])
        b = eng.step(s, [[5], [6]])
        eng.release(s)
        outs.append(torch.cat([a, b]).cpu())
    assert torch.equal(outs[0], outs[1])


def test_padding_and_neighbours_change_nothing(engines, requests_and_truth):
    """The same request alone and next to others of other lengths: float32 logits agree to rounding
    with each other, not only with the oracle."""
    eng = engines("B", "float32")
    prompts, _ = requests_and_truth["B"]
    s = eng.start(1)
    alone = eng.step(s, [prompts[3]], [list(range(len(prompts[3])))]).cpu()
    eng.release(s)
    s = eng.start(3)
    w = [[], list(range(len(prompts[3]))), []]
    among = eng.step(s, [prompts[2], prompts[3], prompts[0]], w).cpu()
    eng.release(s)
    assert float((alone - among).abs().max()) < 1e-5


@pytest.mark.parametrize("host", HOSTS)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(model_folders, plain_models, name, dtype, host):
    import trapetum_b200 as tb
    cfg, w = plain_models[name]
    model = tb.load_model(model_folders[name], dtype, host=host)
    prompts = make_prompts(cfg["vocab_size"], [5, 11, 17, 3], seed=21)
    want = [plain.generate_greedy(cfg, w, p, 12) for p in prompts]
    got = tb.generate(model, prompts, max_tokens=12, max_batch=3)          # two batches: 3 + 1
    if dtype == "float32":
        assert got == want
    else:
        # bfloat16 may part from the oracle at a near-tie; up to there the tokens agree, and the
        # first differing token must be one the oracle also ranks at the top within the error budget
        for p, g, t in zip(prompts, got, want):
            for i, (a, b) in enumerate(zip(g, t)):
                if a != b:
                    logits = plain.forward(cfg, w, p + t[:i])[-1]
                    assert float(logits[b] - logits[a]) < TOLERANCE["of"](name, p + t[:i], dtype) * float(logits.abs().max()), (p, i, a, b)
                    break
    # a stop id ends a request early and is not emitted
    stop = want[0][4]
    cut = tb.generate(model, prompts[:1], max_tokens=12, stop_ids=[stop])[0]
    if dtype == "float32":
        assert cut == want[0][:want[0].index(stop)]


def test_sampled_generation_repeats_and_does_not_depend_on_the_batch(model_folders):
    import trapetum_b200 as tb
    model = tb.load_model(model_folders["A"], "float32")
    prompts = make_prompts(256, [6, 9, 4], seed=33)
    kw = dict(max_tokens=10, temperature=0.9, top_p=0.9, repetition_penalty=1.2, seed=4, stop_ids=[])
    a = tb.generate(model, prompts, max_batch=3, **kw)
    b = tb.generate(model, prompts, max_batch=1, **kw)
    assert a == b and all(len(x) == 10 for x in a)
    assert tb.generate(model, prompts, max_batch=3, **dict(kw, seed=5)) != a


def test_command_line(model_folders, tmp_path, plain_models):
    import numpy as np
    cfg, w = plain_models["A"]
    p = make_prompts(256, [6], seed=2)[0]
    f = tmp_path / "prompt.bin"
    np.asarray(p, dtype="<i4").tofile(f)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gemma_run"), model_folders["A"], str(f),
                          "--dtype", "float32", "--max_tokens", "8"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    line = [l for l in out.stdout.splitlines() if l.startswith("continuation ids:")][0]
    assert eval(line.split(":", 1)[1]) == plain.generate_greedy(cfg, w, p, 8)
    assert "tok/s" in out.stdout and "loaded in" in out.stdout


def test_step_refusals(engines):
    from trapetum_b200.cache import CacheError, CacheFull
    from trapetum_b200.engine import StepError
    eng = engines("A", "float32")
    s = eng.start(2)
    with pytest.raises(StepError, match="vocabulary"):
        eng.step(s, [[1, 2], [256]])
    with pytest.raises(StepError, match="wanted place"):
        eng.step(s, [[1, 2], [3]], [[2], [0]])
    with pytest.raises(StepError, match="at least one token"):
        eng.step(s, [[1], []])
    eng.step(s, [[1, 2], [3]])
    with pytest.raises(StepError, match="exactly one token"):
        eng.step(s, [[1, 2], [3]])
    t = eng.start(1)
    with pytest.raises(StepError, match="all start"):
        eng.step(s + t, [[1], [2], [3]])
    with pytest.raises(StepError, match="twice"):
        eng.step([s[0], s[0]], [[1], [2]])
    eng.release(s + t)
    with pytest.raises(CacheError):
        eng.step(s, [[1], [2]])
    import trapetum_b200 as tb
    small = tb.Engine(eng.model, max_tokens=64)
    u = small.start(1)
    with pytest.raises(CacheFull, match="full"):
        small.step(u, [list(range(65))])
    small.step(u, [list(range(64))])                      # the refused step took nothing
    small.release(u)

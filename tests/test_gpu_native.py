"""The native host (C++ library behind a C interface) against the Python host and the plain implementation:
the same kernels chosen the same way must give the same bits, step by step; its generation loop must emit
the same tokens; the C interface is driven as a C program would drive it; the gemma_run binary runs."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

import plain_gemma2 as plain
from conftest import TINY, TOL, make_prompts, rel_l2, within

pytestmark = pytest.mark.gpu
NAMES = ["A", "B", "C"]
DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_both_hosts_give_the_same_bits(model_folders, plain_models, tolerance_of, name, dtype):
    """Unequal prompts in one step, then one token each for 70 steps (graphs are captured on the way, pages are
    taken, a short request ends early), on both hosts: equal logits, bit for bit, and right against the oracle."""
    import trapetum_b200 as tb
    cfg, w = plain_models[name]
    prompts = make_prompts(cfg["vocab_size"], [130, 41, 99], seed=31)
    truth = [plain.forward(cfg, w, p) for p in prompts]
    cut = [60, 1, 28]
    runs = {}
    for host in tb.HOSTS:
        eng = tb.Engine(tb.load_model(model_folders[name], dtype, host=host), max_tokens=64 * 8)
        for g in eng.cache.groups:
            g.k.fill_(float("nan")); g.v.fill_(float("nan"))
        torch.cuda.synchronize()
        slots = eng.start(3)
        got = [eng.step(slots, [p[:c] for p, c in zip(prompts, cut)], [list(range(c)) for c in cut]).cpu()]
        live = [0, 1, 2]
        for t in range(70):
            gone = [r for r in live if cut[r] + t >= len(prompts[r])]
            for r in gone:
                eng.release([slots[r]])
                live.remove(r)
            got.append(eng.step([slots[r] for r in live], [[prompts[r][cut[r] + t]] for r in live]).cpu())
        eng.release([slots[r] for r in live])
        eng.cache.check()
        assert eng.cache.live_slots() == []
        eng.check_kernels()
        runs[host] = got
    for a, b in zip(runs["python"], runs["native"]):
        assert a.shape == b.shape and torch.equal(a, b)
    first = runs["native"][0]
    o = 0
    for r in range(3):
        worst = max(rel_l2(first[o + i], truth[r][i]) for i in range(cut[r]))
        within(worst, tolerance_of(name, prompts[r], dtype), dtype, f"{name} native host, request {r} prompt")
        o += cut[r]
    within(rel_l2(runs["native"][5][0], truth[0][cut[0] + 4]), tolerance_of(name, prompts[0], dtype), dtype, f"{name} native host, a decoded token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_native_generation_emits_the_python_host_s_tokens(model_folders, plain_models, dtype):
    import trapetum_b200 as tb
    cfg, w = plain_models["A"]
    prompts = make_prompts(cfg["vocab_size"], [5, 11, 17, 3, 70], seed=21)
    models = {h: tb.load_model(model_folders["A"], dtype, host=h) for h in tb.HOSTS}
    greedy = {h: tb.generate(m, prompts, max_tokens=14, max_batch=3, stop_ids=[]) for h, m in models.items()}
    assert greedy["native"] == greedy["python"] and all(len(x) == 14 for x in greedy["native"])
    if dtype == "float32":
        assert greedy["native"] == [plain.generate_greedy(cfg, w, p, 14) for p in prompts]
    kw = dict(max_tokens=12, temperature=0.9, top_p=0.9, repetition_penalty=1.2, seed=4, stop_ids=[])
    sampled = {h: tb.generate(m, prompts, max_batch=4, **kw) for h, m in models.items()}
    assert sampled["native"] == sampled["python"]
    assert tb.generate(models["native"], prompts, max_batch=1, **kw) == sampled["native"]          # batch-independent
    # a stop id ends a request early and is not emitted; the callback sees every emitted token
    stop = greedy["native"][0][4]
    seen = []
    cutoff = tb.generate(models["native"], prompts[:2], max_tokens=14, stop_ids=[stop], on_token=lambda r, t: seen.append((r, t)))
    assert cutoff[0] == greedy["native"][0][:greedy["native"][0].index(stop)]
    assert [t for r, t in seen if r == 0] == cutoff[0] and [t for r, t in seen if r == 1] == cutoff[1]


def test_c_interface_as_a_c_program_would_use_it(model_folders, plain_models):
    """Straight through the exported symbols: load (the spec made natively from config.json), engine, one step with
    the logits copied to the host, generate with a callback, free."""
    from trapetum_b200 import native
    from trapetum_b200.csrc import build
    build.build_all()
    L = native.lib()
    cfg, w = plain_models["A"]
    folder = model_folders["A"].encode()
    L.tb_model_load.restype = ctypes.c_void_p
    model = L.tb_model_load(folder, None, b"float32", 0, None)
    assert model, L.tb_last_error().decode()
    assert L.tb_model_vocab(ctypes.c_void_p(model)) == cfg["vocab_size"]
    L.tb_engine_new.restype = ctypes.c_void_p
    eng = L.tb_engine_new(ctypes.c_void_p(model), ctypes.c_longlong(64 * 4), 0, 1)
    assert eng, L.tb_last_error().decode()
    prompt = make_prompts(cfg["vocab_size"], [23], seed=9)[0]
    I = ctypes.c_int
    slots = (I * 1)()
    assert L.tb_start(ctypes.c_void_p(eng), 1, slots) == 0
    toks = (I * len(prompt))(*prompt)
    n_new = (I * 1)(len(prompt))
    want = (I * 2)(0, len(prompt) - 1)
    n_want = (I * 1)(2)
    out = np.zeros((2, cfg["vocab_size"]), dtype=np.float32)
    rows = I()
    st = L.tb_step_host(ctypes.c_void_p(eng), slots, 1, toks, n_new, want, n_want, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                        ctypes.c_longlong(out.size), ctypes.byref(rows))
    assert st == 0 and rows.value == 2, L.tb_last_error().decode()
    truth = plain.forward(cfg, w, prompt)
    assert rel_l2(torch.from_numpy(out[0]), truth[0]) < 1e-5 and rel_l2(torch.from_numpy(out[1]), truth[-1]) < 1e-5
    # a step that is no step is refused with its own status and a message, and takes nothing
    bad = (I * 2)(1, 2)
    two = (I * 1)(2)
    assert L.tb_step_host(ctypes.c_void_p(eng), slots, 1, bad, two, None, None, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                          ctypes.c_longlong(out.size), ctypes.byref(rows)) == 2
    assert b"exactly one token" in L.tb_last_error()
    assert L.tb_release(ctypes.c_void_p(eng), slots, 1) == 0
    assert L.tb_release(ctypes.c_void_p(eng), slots, 1) != 0                      # freed twice: an error, not a crash
    # generation with a per-token callback
    seen = []
    cb = native._ON_TOKEN(lambda r, t, u: seen.append((r, t)) or 0)
    params = native._Sampling(0.0, 0.95, 1.0, 8, 0)
    lens = (I * 1)(len(prompt))
    got = (I * 8)()
    got_n = (I * 1)()
    st = L.tb_generate(ctypes.c_void_p(eng), toks, lens, 1, ctypes.byref(params), None, -1, 8, cb, None, got, got_n, 8)
    assert st == 0, L.tb_last_error().decode()
    want_ids = plain.generate_greedy(cfg, w, prompt, 8)
    assert list(got[:got_n[0]]) == want_ids and [t for _, t in seen] == want_ids
    assert L.tb_kernel_errors(ctypes.c_void_p(eng)) == b""
    L.tb_engine_free(ctypes.c_void_p(eng))
    L.tb_model_free(ctypes.c_void_p(model))
    # errors of loading come back as messages
    assert not L.tb_model_load(b"/nonexistent", None, b"float32", 0, None)
    assert b"config.json" in L.tb_last_error()


def test_gemma_run_binary(model_folders, plain_models, tmp_path):
    from trapetum_b200.csrc import build
    build.build_all()
    cfg, w = plain_models["A"]
    p = make_prompts(256, [6], seed=2)[0]
    f = tmp_path / "prompt.bin"
    np.asarray(p, dtype="<i4").tofile(f)
    out = subprocess.run([build.native_binary_path(), model_folders["A"], str(f), "--dtype", "float32", "--max_tokens", "8"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    line = [l for l in out.stdout.splitlines() if l.startswith("continuation ids:")][0]
    assert eval(line.split(":", 1)[1]) == plain.generate_greedy(cfg, w, p, 8)
    assert "tok/s" in out.stdout and "loaded in" in out.stdout
    bad = subprocess.run([build.native_binary_path(), str(tmp_path), str(f)], capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "config.json" in bad.stderr


def test_native_random_model_is_the_folder_s_model(tmp_path):
    import trapetum_b200 as tb
    from conftest import TINY_B
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_B, 11, 0.03, 0.2, device="cpu")
    prompts = [[5, 9, 200, 3, 77], [1]]
    outs = []
    for m in (tb.load_model(d, "bfloat16", host="native"), tb.random_model(TINY_B, 11, 0.03, 0.2, "bfloat16", host="native")):
        eng = tb.Engine(m, max_tokens=128)
        s = eng.start(2)
        outs.append(eng.step(s, prompts, [[0, 4], [0]]).cpu())
        eng.release(s)
    assert torch.equal(outs[0], outs[1])

"""bin/trace_run as a user runs it: a subprocess, steps on standard input, logits in files."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_gemma2 as plain
from conftest import ROOT, TOL, make_prompts, rel_l2, within

pytestmark = pytest.mark.gpu


def run_trace(folder, dtype, out, steps, max_tokens, host=None):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out, "--max-tokens", str(max_tokens)] + (["--host", host] if host else []),
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.split() == [x for s in steps for x in ("done", str(s["step"]))]
    return proc


@pytest.mark.parametrize("host", [None, "python"])          # the program's own choice (the native host), and the Python host
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_three_ways(model_folders, plain_models, tolerance_of, tmp_path, name, dtype, host):
    cfg, w = plain_models[name]
    V = cfg["vocab_size"]
    reqs = make_prompts(V, [40, 75, 130], seed=3)
    truth = [plain.forward(cfg, w, r) for r in reqs]
    steps, expect = [], {}

    def add(entries, end=()):
        n = len(steps)
        steps.append({"step": n, "entries": entries, "end": list(end)})
        return n
    # 1. each request alone and whole
    for i, r in enumerate(reqs):
        n = add([{"id": f"w{i}", "tokens": r, "want": list(range(len(r)))}], end=[f"w{i}"])
        expect[n] = truth[i]
    # 2. whole but for the last 32 tokens, then those one by one
    for i, r in enumerate(reqs):
        k = len(r) - 32
        n = add([{"id": f"t{i}", "tokens": r[:k], "want": [k - 1]}])
        expect[n] = truth[i][k - 1:k]
        for j in range(k, len(r)):
            n = add([{"id": f"t{i}", "tokens": [r[j]], "want": [0]}], end=[f"t{i}"] if j == len(r) - 1 else [])
            expect[n] = truth[i][j:j + 1]
    # 3. an unequal batch whose shorter requests end earlier, twice, so that slots are used again;
    #    some steps want nothing
    for rep in range(2):
        cut = [7, 60, 33]
        ids = [f"b{rep}_{i}" for i in range(3)]
        n = add([{"id": ids[i], "tokens": reqs[i][:cut[i]], "want": [0, cut[i] - 1]} for i in range(3)])
        expect[n] = torch.cat([truth[i][[0, cut[i] - 1]] for i in range(3)])
        t = 0
        live = [0, 1, 2]
        while live:
            nxt = [i for i in live if cut[i] + t + 1 < len(reqs[i])]
            quiet = (t % 5 == 3)
            n = add([{"id": ids[i], "tokens": [reqs[i][cut[i] + t]], "want": [] if quiet else [0]} for i in live],
                    end=[ids[i] for i in live if i not in nxt])
            if not quiet:
                expect[n] = torch.stack([truth[i][cut[i] + t] for i in live])
            live = nxt
            t += 1
    out = str(tmp_path / "out")
    # 3 pages + 2 pages + 1 page live at most (the batch), the single requests need less
    run_trace(model_folders[name], dtype, out, steps, max_tokens=64 * 6, host=host)
    files = sorted(os.listdir(out))
    assert files == sorted(f"{n}.f32" for n in expect)
    for n, want in expect.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V))
        assert got.shape == want.shape
        worst = max(rel_l2(got[i], want[i]) for i in range(got.shape[0]))
        tol = max(tolerance_of(name, reqs[int(e["id"][-1])], dtype) for e in steps[n]["entries"])
        within(worst, tol, dtype, f"{name} replay step {n} ({steps[n]['entries'][0]['id']}...)")


def test_replay_refuses_what_does_not_fit(model_folders, tmp_path):
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": list(range(100)), "want": []}], "end": []}]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folders["A"],
                           "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                          input=json.dumps(steps[0]) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "cache is full" in proc.stderr

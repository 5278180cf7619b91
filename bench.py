#!/usr/bin/env python3
"""Benchmark: decode tokens per second of Gemma-2-shaped models with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 2b|9b|27b] [--batch 8] [--context 8192] [--layers L]
    python bench.py --impl reference ...        # the reference arm: not installable here

A step is one decode step: one new token for each of ``batch`` sequences whose caches hold about
``context`` tokens.  Prints ONE JSON line.  ``value`` is timed on the device with CUDA events around
K steps, as the median of five such regions (``spread`` gives the least and the most, and each region's
median SM clock); ``e2e`` runs the same steps through the public Python API with host token lists in and
host token ids out (a pinned host-to-device copy of the step's inputs and a device-to-host read of the
chosen tokens every step).  ``prefill`` times one 2,048-token prompt; ``roofline`` sets the bytes a decode
step has to read (every weight once, the live requests' cache) against its time; ``points`` repeats the
decode measurement at batch 1 and 64; ``runs`` holds the other measurements that the three model shapes
are quoted on (caches of 2,048 tokens, the 9B shape's unequal batch of 8, the 27B shape from 2,048-token
prompts, each shape's prefill), every one with its bytes or FLOPs, its time and its fraction of the peak.
Weights are made on the device by the counter-based generator (``tb.random_model``).  Peaks come from
MEASURED_PEAKS.json beside this file when the driver wrote it, otherwise from the fallback figures
(6.65 TB/s, 1.59 PFLOP/s).

This library runs on one GPU: for --gpus > 1 it says so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

def _shape(L, H, nh, nkv, hd, I, qpas):
    return {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "num_hidden_layers": L, "hidden_size": H,
            "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": I,
            "vocab_size": 256000, "rope_theta": 10000.0, "sliding_window": 4096, "query_pre_attn_scalar": qpas,
            "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6,
            "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "max_position_embeddings": 8192}


# Layer sizes of Gemma-2-2B, -9B and -27B; weights are random (seeds 2, 3, 4).
MODELS = {"2b": _shape(26, 2304, 8, 4, 256, 9216, 256), "9b": _shape(42, 3584, 16, 8, 256, 14336, 256),
          "27b": _shape(46, 4608, 32, 16, 128, 36864, 144)}
SEEDS = {"2b": 2, "9b": 3, "27b": 4}
GEMMA2_2B = MODELS["2b"]
PREFILL_TOKENS = 2048
REPEATS = 5              # timed regions per measurement; the median is reported


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons (NVML, else nvidia-smi) while a timed region runs.  Reads only."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.stamps, self._stop, self._t = [], [], threading.Event(), None

    def _run_nvml(self) -> bool:
        """Reads the same values through NVML every 5 ms (an nvidia-smi call takes longer than a short timed
        region); False if NVML cannot be used here."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(0)
            top = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), reasons(h)
        except Exception:
            return False
        bits = (0x8, 0x40, 0x20, 0x4)          # hw_slowdown, hw_thermal_slowdown, sw_thermal_slowdown, sw_power_cap
        while not self._stop.is_set():
            try:
                mhz, mask = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), int(reasons(h))
                self.rows.append([str(mhz), str(top)] + ["Active" if mask & b else "Not Active" for b in bits])
                self.stamps.append(time.perf_counter())
            except Exception:
                pass
            self._stop.wait(0.005)
        return True

    def _run(self):
        if self._run_nvml():
            return
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    self.rows.append([x.strip() for x in out[0].split(",")])
                    self.stamps.append(time.perf_counter())
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def mhz_between(self, t0, t1):
        """Median SM clock of the samples taken between two host times (None if there is none)."""
        m = sorted(int(r[0]) for r, t in zip(self.rows, self.stamps) if t0 <= t <= t1 and r[0].isdigit())
        return m[len(m) // 2] if m else None

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no samples"]}
        mhz = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(self.rows[0][1]) if self.rows[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(self.rows)}


HOST = None              # which host runs the models (None: the library's default, the native host for these models)


def build_model(cfg, seed):
    import trapetum_b200 as tb
    return tb.random_model(cfg, seed, 0.02, 0.1, "bfloat16", "cuda:0", host=HOST)


def launches():
    """Kernel launches of this process so far, on whichever host runs the steps."""
    import sys as _sys
    from trapetum_b200.csrc import ops
    nat = _sys.modules.get("trapetum_b200.native")
    return ops.launches() + (nat.launches() if nat is not None and nat._lib is not None else 0)


def weight_bytes(cfg):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (qd + 2 * kvd) * H + H * qd + 2 * I * H + H * I + 4 * H
    return 2 * (L * per_layer + V * H + H)          # the embedding table is read once, as the output head


def cache_bytes(cfg, ctx):
    """Key and value bytes one sequence with ``ctx`` tokens makes a decode step read."""
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    W = cfg["sliding_window"]
    total = 0
    for i in range(cfg["num_hidden_layers"]):
        rows = min(ctx, W) if i % 2 == 0 else ctx
        total += rows * kvd * 2 * 2
    return total


def prefill_flops(cfg, lens):
    """FLOPs of one step that brings whole prompts of these lengths (the head runs on each last position)."""
    if isinstance(lens, int):
        lens = [lens]
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    lin = 2 * sum(lens) * ((qd + 2 * kvd) * H + H * qd + 2 * I * H + H * I)
    W = cfg["sliding_window"]
    att = 0
    for i in range(L):
        for T in lens:
            if i % 2 == 0 and T > W:
                pairs = W * (W + 1) // 2 + (T - W) * W
            else:
                pairs = T * (T + 1) // 2
            att += 4 * qd * pairs
    return L * lin + att + 2 * V * H * len(lens)


def fill_cache(engine, lens):
    """Sequences whose caches hold ``lens`` tokens of random keys and values (no prefill is run:
    the decode step's work does not depend on what the keys are)."""
    slots = engine.start(len(lens))
    engine.cache.grow({s: n for s, n in zip(slots, lens)})
    return slots


def time_decode(engine, torch, ctxs, steps, warmup, vocab, repeats=REPEATS, e2e=False, clocks=None):
    """Decode steps of a batch whose caches hold about ``ctxs`` tokens (one number per sequence; they end the
    measurement at these lengths).  ``repeats`` regions of ``steps`` steps each are timed with CUDA events.
    Returns a dict: ms (median per step), ms_min, ms_max, regions [{ms, sm_mhz}], mean_ctx (per sequence, over
    the timed steps), launches (per step), and with ``e2e`` also e2e_ms and h2d."""
    from trapetum_b200.csrc import ops
    batch = len(ctxs)
    g = torch.Generator().manual_seed(batch)
    total = warmup + repeats * steps + (2 * warmup + steps if e2e else 0)
    start = [max(1, c - total) for c in ctxs]
    slots = fill_cache(engine, start)
    out = {}
    try:
        toks = torch.randint(0, vocab, (total + 2, batch), generator=g).tolist()
        it = iter(toks)
        for _ in range(warmup):
            engine.step(slots, [[t] for t in next(it)], borrow=True)
        torch.cuda.synchronize()
        regions, done = [], warmup
        n0 = launches()
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e0.record()
            for _ in range(steps):
                engine.step(slots, [[t] for t in next(it)], borrow=True)
            e1.record()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            regions.append({"ms": round(e0.elapsed_time(e1) / steps, 4),
                            "sm_mhz": clocks.mhz_between(t0, t1) if clocks is not None else None})
        out["launches"] = (launches() - n0) // (repeats * steps)
        ms = sorted(r["ms"] for r in regions)
        out.update(ms=ms[len(ms) // 2], ms_min=ms[0], ms_max=ms[-1], regions=regions)
        # the context each timed step reads: the tokens before it, and its own
        first = [s0 + warmup + 1 for s0 in start]
        out["mean_ctx"] = [f + (repeats * steps - 1) / 2.0 for f in first]
        if e2e:
            # end to end: host token lists in, chosen token ids out, each step feeding the next
            cur = next(it)
            for _ in range(warmup):
                cur = engine.step_tokens(slots, [[t] for t in cur])
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                cur = engine.step_tokens(slots, [[t] for t in cur])
            torch.cuda.synchronize()
            out["e2e_ms"] = (time.perf_counter() - t0) * 1e3 / steps
            out["h2d"] = engine.last_h2d_bytes
        return out
    finally:
        engine.release(slots)


def time_generate(engine, torch, ctx, batch, steps, warmup, vocab):
    """Decode steps through the generation entry point (``tb.generate``: host prompts in, host tokens out through the
    per-token callback): prompts that fill the caches to about ``ctx`` tokens, then ``warmup + steps`` new tokens
    each; the times between the callbacks of a request's tokens give ms per step: (median, mean).  Every step
    copies its inputs from pinned host memory and its chosen ids back to the host.  The median is the steady step:
    right after the prompts' own step (tens of thousands of tokens on the tensor cores at the power cap) the clocks
    stay low for some tens of milliseconds, which the mean of a short run shows and the median does not."""
    import trapetum_b200 as tb
    g = torch.Generator().manual_seed(1000 + batch)
    warmup = warmup + 100          # the clocks need about 120 ms to come back after the prompts' step: those steps are not timed
    n_new = warmup + steps + 1
    prompts = torch.randint(0, vocab, (batch, max(1, ctx - n_new)), generator=g).tolist()
    stamps = []

    def on_token(request, token):
        if request == 0:
            stamps.append(time.perf_counter())
    tb.generate(engine, prompts, max_tokens=n_new, stop_ids=[], max_batch=batch, on_token=on_token)
    torch.cuda.synchronize()
    gaps = sorted((b - a) * 1e3 for a, b in zip(stamps[warmup:], stamps[warmup + 1:]))
    return gaps[len(gaps) // 2], (stamps[-1] - stamps[warmup]) * 1e3 / (len(stamps) - 1 - warmup)


def decode_record(cfg, r, hbm_gbs):
    """What a decode measurement says against the memory roofline."""
    nbytes = weight_bytes(cfg) + sum(cache_bytes(cfg, int(round(c))) for c in r["mean_ctx"])
    gbs = nbytes / (r["ms"] * 1e-3) / 1e9
    return {"value": round(len(r["mean_ctx"]) * 1e3 / r["ms"], 1), "unit": "tokens/s", "ms": r["ms"],
            "ms_min": r["ms_min"], "ms_max": r["ms_max"], "bytes": nbytes, "gbs": round(gbs, 1),
            "frac": round(gbs / hbm_gbs, 4)}


def time_prefill(engine, torch, lens, vocab, reps, warmup):
    """One step that brings whole prompts of ``lens`` tokens: (median ms on the device, median ms of host time
    to issue the step, median ms from the call to the logits' arrival on the host)."""
    if isinstance(lens, int):
        lens = [lens]
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    dev, host, whole = [], [], []
    for i in range(warmup + reps):
        s = engine.start(len(lens))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        logits = engine.step(s, prompts, borrow=True)
        e1.record()
        t1 = time.perf_counter()
        logits[:, :8].cpu()
        t2 = time.perf_counter()
        torch.cuda.synchronize()
        engine.release(s)
        if i >= warmup:
            dev.append(e0.elapsed_time(e1)); host.append((t1 - t0) * 1e3); whole.append((t2 - t0) * 1e3)
    med = lambda v: sorted(v)[len(v) // 2]
    return med(dev), med(host), med(whole)


def prefill_record(cfg, lens, ms, host_ms, e2e_ms, bf16_tflops):
    lens = [lens] if isinstance(lens, int) else lens
    fl = prefill_flops(cfg, lens)
    return {"value": round(sum(lens) * 1e3 / ms, 1), "unit": "tokens/s", "tokens": sum(lens), "ms": round(ms, 3),
            "host_ms": round(host_ms, 3), "e2e_ms": round(e2e_ms, 3), "flops": fl,
            "frac": round(fl / (ms * 1e-3) / (bf16_tflops * 1e12), 4)}


def random_cache(engine):
    for g in engine.cache.groups:                         # random keys and values, small enough for a sane softmax
        g.k.normal_(0.0, 0.5)
        g.v.normal_(0.0, 0.5)


def other_runs(torch, which, steps, warmup, hbm_gbs, bf16_tflops, have=None):
    """The measurements beside the headline: per model shape, decode at batch 1/8/64 with caches of 2,048 tokens
    (the 9B shape: its unequal batch of 8, prompts U[64, 2048], decode and the prompts' own step), and a
    2,048-token prompt.  ``have``: (name, model) already built.  Models are built and freed one after another."""
    from trapetum_b200 import Engine
    runs = {}
    for name in which:
        cfg = MODELS[name]
        V = cfg["vocab_size"]
        model = have[1] if have and have[0] == name else build_model(cfg, SEEDS[name])
        engine = Engine(model, max_tokens=64 * 2112, max_slots=64)
        random_cache(engine)
        st = max(8, steps // 2)
        for b in (1, 8, 64):
            r = time_decode(engine, torch, [2048] * b, st, warmup, V, repeats=3)
            runs[f"{name}_decode_b{b}_ctx2048"] = decode_record(cfg, r, hbm_gbs)
        if name == "9b":
            lens = torch.randint(64, 2049, (8,), generator=torch.Generator().manual_seed(3)).tolist()
            r = time_decode(engine, torch, lens, st, warmup, V, repeats=3)
            rec = decode_record(cfg, r, hbm_gbs)
            rec["prompt_lens"] = " ".join(map(str, lens))
            runs["9b_decode_unequal_b8"] = rec
            runs["9b_prefill_unequal_b8"] = prefill_record(cfg, lens, *time_prefill(engine, torch, lens, V, 3, 3), bf16_tflops)
        if name != "2b":
            runs[f"{name}_prefill_{PREFILL_TOKENS}"] = prefill_record(
                cfg, PREFILL_TOKENS, *time_prefill(engine, torch, PREFILL_TOKENS, V, 3, 3), bf16_tflops)
        del engine, model
        have = None
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    return runs


def leave_out_report(engine, model, cfg, torch, args, warmup) -> int:
    """What each kind of launch costs inside the step's graph: the step is timed whole, then with that kind
    replaced by a stand-in that launches nothing and returns a buffer of the right shape."""
    from trapetum_b200.csrc import ops
    from trapetum_b200.engine import Engine
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    real = {k: getattr(ops, k) for k in ("attn_decode", "add_rmsnorm", "gemm_tc")}
    bufs = {}

    def buf(key, shape, dtype):
        k = (key, tuple(shape), dtype)
        if k not in bufs:
            bufs[k] = torch.zeros(shape, dtype=dtype, device="cuda:0")
        return bufs[k]

    def no_attn(q, *a, **kw):
        rows = q.shape[1] if q.dim() == 3 else q.shape[0]
        return buf("attn", (rows, qd), torch.bfloat16)

    def no_norm(h, a, wa, ea, oa, wb=None, eps_b=0.0, off_b=0.0, out_dtype=None):
        return buf("norm", h.shape, out_dtype) if wb is not None else None

    def no_gemm(shape):
        def f(a, w, out_dtype, softcap=0.0, splits=None, out=None, partials=False, gated_act=None):
            if tuple(w.shape) != shape:
                return real["gemm_tc"](a, w, out_dtype, softcap, splits, out, partials, gated_act)
            M, N = a.shape[0], w.shape[0]
            if gated_act:
                return buf("g", (M, N // 2), torch.bfloat16)
            return buf("p", (1, M, N), torch.float32) if partials else buf("o", (M, N), out_dtype)
        return f

    kinds = {"nothing": {}, "attention": {"attn_decode": no_attn}, "add_rmsnorm": {"add_rmsnorm": no_norm},
             "gemm qkv": {"gemm_tc": no_gemm((qd + 2 * kvd, H))}, "gemm o": {"gemm_tc": no_gemm((H, qd))},
             "gemm gate_up": {"gemm_tc": no_gemm((2 * I, H))}, "gemm down": {"gemm_tc": no_gemm((H, I))},
             "gemm head": {"gemm_tc": no_gemm((V, H))}}
    whole = None
    try:
        for name, patch in kinds.items():
            for k, v in real.items():
                setattr(ops, k, v)
            for k, v in patch.items():
                setattr(ops, k, v)
            eng = Engine(model, max_tokens=args.batch * args.context, max_slots=args.batch)
            r = time_decode(eng, torch, [args.context] * args.batch, args.steps, warmup, V, repeats=1)
            ms, launches = r["ms"], r["launches"]
            whole = ms if whole is None else whole
            print(json.dumps({"left_out": name, "ms_per_step": round(ms, 4), "launches": launches,
                              "saves_us": round((whole - ms) * 1e3, 1),
                              "saves_us_per_layer": round((whole - ms) * 1e3 / args.layers, 2)}), flush=True)
            del eng
    finally:
        for k, v in real.items():
            setattr(ops, k, v)
    return 0


def gemm_compare(cfg, torch, tokens, bf16_tflops):
    """The four products of a layer at ``tokens`` tokens, this library's tensor-core kernel beside torch.matmul
    (cuBLAS), as a comparison only: neither result feeds a bench number.  Each launch gets another of three weight
    matrices, so the weights come from memory; 12 launches are captured in a CUDA graph and timed as one."""
    from trapetum_b200.csrc import ops
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    shapes = [("qkv", qd + 2 * kvd, H), ("o", H, qd), ("gate_up", 2 * I, H), ("down", H, I)]
    g0 = torch.Generator(device="cuda").manual_seed(1)

    def timed(fn, reps=12):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                fn(i)
        best = None
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); graph.replay(); e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) / reps
            best = t if best is None else min(best, t)
        return best

    for name, N, K in shapes:
        a = (torch.randn(tokens, K, device="cuda", generator=g0) * 0.5).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device="cuda", generator=g0) * 0.05).to(torch.bfloat16) for _ in range(3)]
        outs = [torch.empty(tokens, N, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
        ours = timed(lambda i: ops.gemm_tc(a, ws[i % 3], torch.bfloat16))
        lib = timed(lambda i: torch.matmul(a, ws[i % 3].t(), out=outs[i % 3]))
        fl = 2.0 * tokens * N * K
        print(json.dumps({"product": name, "tokens": tokens, "weight_rows": N, "k": K,
                          "ours_us": round(ours * 1e3, 1), "ours_tflops": round(fl / ours / 1e9, 1),
                          "torch_matmul_us": round(lib * 1e3, 1), "torch_matmul_tflops": round(fl / lib / 1e9, 1),
                          "ours_over_torch": round(lib / ours, 3),
                          "ours_frac_of_peak": round(fl / (ours * 1e-3) / (bf16_tflops * 1e12), 3)}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="2b", choices=sorted(MODELS), help="the headline's model shape")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has (same layer sizes); both numbers are reported")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points, the prefill and the other runs")
    ap.add_argument("--no-e2e", action="store_true",
                    help="skip the end-to-end run through tb.generate (it starts with 8 prompts of about 8,000 tokens); the "
                         "step-loop figure then stands in its place (for short captures under a profiler)")
    ap.add_argument("--runs", default="2b,9b,27b",
                    help="model shapes whose other measurements (caches of 2,048 tokens, prefill) are taken: a comma "
                         "list out of 2b, 9b, 27b, or 'none'")
    ap.add_argument("--host", default=None, choices=["native", "python"],
                    help="the host that runs the steps (default: the library's own choice, the native host)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="instead of the bench line: time only the prompt of 2,048 tokens and print one line about it")
    ap.add_argument("--leave-out", action="store_true",
                    help="instead of the bench line: the decode step re-timed with one kind of launch left out at a "
                         "time (its results are then wrong; only its time is of interest), one line per kind")
    ap.add_argument("--gemm-compare", type=int, default=0, metavar="TOKENS",
                    help="instead of the bench line: the four products of a layer of --model at TOKENS tokens, this "
                         "library's kernel beside torch.matmul, one line per product (a comparison only)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "neuralboot/trapetum is a Rust crate (no setup.py or pyproject.toml: pip reports 'not "
                          "installable'); no cargo/rustc in this image, and its Gemma-2 path runs 4-bit codebook "
                          "weights only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: trapetum_b200 is a single-GPU library; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    warmup = max(3, args.warmup)

    import torch
    if args.gemm_compare:
        return gemm_compare(MODELS[args.model], torch, args.gemm_compare, peaks()[1])
    from trapetum_b200 import Engine
    global HOST
    HOST = "python" if args.leave_out else args.host
    full = MODELS[args.model]
    args.layers = args.layers or full["num_hidden_layers"]
    cfg = dict(full, num_hidden_layers=args.layers)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    model = build_model(cfg, SEEDS[args.model])
    V = cfg["vocab_size"]
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    per_token = 4 * cfg["num_key_value_heads"] * cfg["head_dim"] * cfg["num_hidden_layers"]      # key and value bytes
    if max_batch > args.batch and max_batch * args.context * per_token + weight_bytes(cfg) > 150e9:
        max_batch = args.batch                            # the batch-64 point does not fit beside these weights
    engine = Engine(model, max_tokens=max_batch * args.context, max_slots=max(max_batch, args.batch))
    random_cache(engine)

    if args.leave_out:
        return leave_out_report(engine, model, cfg, torch, args, warmup)
    if args.prefill_only:
        pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=max(1, args.steps), warmup=warmup)
        print(json.dumps({"prefill_ms": round(pms, 3), "host_ms": round(hms, 3), "e2e_ms": round(wms, 3),
                          "tokens": PREFILL_TOKENS, "layers": args.layers,
                          "frac": round(prefill_flops(cfg, PREFILL_TOKENS) / (pms * 1e-3) / (bf16_tflops * 1e12), 4),
                          "of": peak_src}))
        return 0

    with ClockSampler() as clocks:
        r = time_decode(engine, torch, [args.context] * args.batch, args.steps, warmup, V, e2e=True, clocks=clocks)
    dev_ms, loop_ms = r["ms"], r["e2e_ms"]
    e2e_ms = e2e_mean_ms = loop_ms                     # replaced below by the run through tb.generate
    rec = decode_record(cfg, r, hbm_gbs)
    csum = clocks.summary()
    mhz = csum.get("sm_mhz")

    out = {
        "metric": "decode tok/s at batch %d (Gemma-2-%s)" % (args.batch, args.model.upper()),
        "value": rec["value"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights seed %d made on the device, uniform token ids, random "
                                 "cache contents)" % SEEDS[args.model],
        "config": {"model": "gemma-2-%s-shape" % args.model, "global_batch": args.batch, "seq_len": args.context,
                   "parallelism": "1 gpu", "layers": args.layers, "layers_of_model": full["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "window": cfg["sliding_window"],
                   "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (each step reads every weight)",
                   "timed": "median of %d regions of %d steps" % (REPEATS, args.steps), "peaks": peak_src,
                   "host": type(engine).__module__.split(".")[-1].replace("engine", "python")},
        "clocks": csum,
        "spread": {"ms_min": r["ms_min"], "ms_max": r["ms_max"], "regions": r["regions"],
                   "ms_x_ghz": round(dev_ms * mhz / 1e3, 4) if mhz else None},
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": 4 * args.batch,
                "how": "engine.step_tokens in a loop: host tokens in, the chosen tokens back on the host, every step",
                "mean_ms_per_step": round(e2e_mean_ms, 4),
                "step_loop_value": round(args.batch * 1e3 / loop_ms, 1), "step_loop_ms": round(loop_ms, 4)},
        "gpu_launches": r["launches"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": rec["gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": rec["frac"], "of": peak_src, "bytes_per_step": rec["bytes"]},
    }
    if not args.no_points:
        pts, runs = {}, {}
        for b in (1, 64):
            if b > engine.cache.max_slots:
                continue
            rb = time_decode(engine, torch, [args.context] * b, max(8, args.steps // 2), warmup, V, repeats=3, e2e=(b == 1))
            rr = decode_record(cfg, rb, hbm_gbs)
            pts[f"decode_b{b}"] = rr["value"]
            if b == 1:
                pts["e2e_b1_step_loop"] = round(1e3 / rb["e2e_ms"], 1)
            runs[f"{args.model}_decode_b{b}_ctx{args.context}"] = rr
        pms, hms, wms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=5, warmup=3)
        prec = prefill_record(cfg, PREFILL_TOKENS, pms, hms, wms, bf16_tflops)
        out["prefill"] = dict(prec, of=peak_src)
        out["points"] = pts
        if not args.no_e2e:
            pts["e2e_b1"] = round(1e3 / time_generate(engine, torch, args.context, 1, max(8, args.steps // 2), warmup, V)[0], 1)
        if not args.no_e2e:
            e2e_ms, e2e_mean_ms = time_generate(engine, torch, args.context, args.batch, args.steps, warmup, V)
            out["e2e"].update(value=round(args.batch * 1e3 / e2e_ms, 1), ms_per_step=round(e2e_ms, 4),
                              mean_ms_per_step=round(e2e_mean_ms, 4),
                              how="tb.generate: host prompts in, tokens out through its callback; median time between a "
                                  "request's tokens, the first hundred after the prompts' step left out")
        which = [] if args.runs == "none" else [w for w in args.runs.split(",") if w in MODELS]
        if args.layers != full["num_hidden_layers"]:
            which = []                                  # the other runs are of whole models
        del engine
        torch.cuda.empty_cache()
        have = (args.model, model)
        del model
        runs.update(other_runs(torch, which, args.steps, warmup, hbm_gbs, bf16_tflops, have))
        for k, v in runs.items():
            if "decode" in k:
                pts.setdefault(k, v["value"])
        out["runs"] = runs
    from trapetum_b200.csrc import ops
    err = ops.kernel_errors()
    if err:
        out["error"] = f"a bounded wait ran out: {err}"
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())

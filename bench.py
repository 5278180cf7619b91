#!/usr/bin/env python3
"""Benchmark: decode tokens per second of a Gemma-2-2B-shaped model with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers L]
    python bench.py --impl reference ...        # the reference arm: not installable here

A step is one decode step: one new token for each of ``batch`` sequences whose caches hold about
``context`` tokens.  Prints ONE JSON line.  ``value`` is timed on the device with CUDA events around
K steps; ``e2e`` runs the same steps through the public Python API with host token lists in and host
token ids out (a pinned host-to-device copy of the step's inputs and a device-to-host read of the
chosen tokens every step).  ``prefill`` times one 2,048-token prompt; ``roofline`` sets the bytes a
decode step has to read (every weight once, the live requests' cache) against its time; ``points``
repeats the decode measurement at batch 1 and 64.  Peaks come from MEASURED_PEAKS.json beside this
file when the driver wrote it, otherwise from the fallback figures (6.65 TB/s, 1.59 PFLOP/s).

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

# Layer sizes of Gemma-2-2B; weights are random (seed 2).
GEMMA2_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 26, "hidden_size": 2304, "num_attention_heads": 8, "num_key_value_heads": 4,
    "head_dim": 256, "intermediate_size": 9216, "vocab_size": 256000, "rope_theta": 10000.0,
    "sliding_window": 4096, "query_pre_attn_scalar": 256, "attn_logit_softcapping": 50.0,
    "final_logit_softcapping": 30.0, "rms_norm_eps": 1e-6, "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True, "max_position_embeddings": 8192,
}
PREFILL_TOKENS = 2048


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
        self.rows, self._stop, self._t = [], threading.Event(), None

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

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi gave no samples"]}
        mhz = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(self.rows[0][1]) if self.rows[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(self.rows)}


def build_model(cfg, seed):
    import torch

    import trapetum_b200 as tb
    from trapetum_b200.config import load_config
    from trapetum_b200.csrc import build
    from trapetum_b200.engine.model import Model
    from trapetum_b200.parts import Runtime
    from trapetum_b200.weights.loader import random_tensors
    _, spec = load_config(cfg)
    model = Model(spec, Runtime(torch.bfloat16, torch.device("cuda:0")))
    build.require(model.kernel_files())
    tensors = dict(random_tensors(model.tensor_specs(), seed, 0.02, 0.1, device="cuda:0"))
    model.bind(tensors)
    return model


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


def prefill_flops(cfg, T):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    qd, kvd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    lin = 2 * T * ((qd + 2 * kvd) * H + H * qd + 2 * I * H + H * I)
    W = cfg["sliding_window"]
    att = 0
    for i in range(L):
        pairs = sum(min(t + 1, W) if i % 2 == 0 else t + 1 for t in range(T))
        att += 4 * qd * pairs
    return L * lin + att + 2 * V * H               # the head runs on the last position only


def fill_cache(engine, n, ctx):
    """``n`` sequences whose caches hold ``ctx`` tokens of random keys and values (no prefill is run:
    the decode step's work does not depend on what the keys are)."""
    slots = engine.start(n)
    engine.cache.grow({s: ctx for s in slots})
    return slots


def time_decode(engine, torch, batch, ctx, steps, warmup, vocab, sampler=None):
    """(ms per step on the device, ms per step end to end, launches per step, h2d bytes per step)."""
    from trapetum_b200.csrc import ops
    g = torch.Generator().manual_seed(batch)
    slots = fill_cache(engine, batch, ctx - (warmup + steps) * 2 - 4)
    try:
        toks = torch.randint(0, vocab, (2 * (warmup + steps) + 4, batch), generator=g).tolist()
        it = iter(toks)
        for _ in range(warmup):
            engine.step(slots, [[t] for t in next(it)], borrow=True)
        torch.cuda.synchronize()
        n0 = ops.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            engine.step(slots, [[t] for t in next(it)], borrow=True)
        e1.record()
        torch.cuda.synchronize()
        dev_ms = e0.elapsed_time(e1) / steps
        launches = (ops.launches() - n0) // steps
        # end to end: host token lists in, chosen token ids out, each step feeding the next
        cur = next(it)
        for _ in range(warmup):
            cur = engine.step(slots, [[t] for t in cur], borrow=True, greedy=True).cpu().tolist()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            cur = engine.step(slots, [[t] for t in cur], borrow=True, greedy=True).cpu().tolist()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
        shape = next((d for key, d in engine._decode.items() if key[0] == batch), None)
        h2d = shape.h2d_bytes if shape is not None else 0
        return dev_ms, e2e_ms, launches, h2d
    finally:
        engine.release(slots)


def time_prefill(engine, torch, T, vocab, reps, warmup):
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, vocab, (T,), generator=g).tolist()
    times = []
    for i in range(warmup + reps):
        s = engine.start(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step(s, [prompt], borrow=True)
        e1.record()
        torch.cuda.synchronize()
        engine.release(s)
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


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
            ms, _, launches, _ = time_decode(eng, torch, args.batch, args.context, args.steps, warmup, V)
            whole = ms if whole is None else whole
            print(json.dumps({"left_out": name, "ms_per_step": round(ms, 4), "launches": launches,
                              "saves_us": round((whole - ms) * 1e3, 1),
                              "saves_us_per_layer": round((whole - ms) * 1e3 / args.layers, 2)}), flush=True)
            del eng
    finally:
        for k, v in real.items():
            setattr(ops, k, v)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=GEMMA2_2B["num_hidden_layers"],
                    help="fewer layers than the model has (same layer sizes); both numbers are reported")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--prefill-only", action="store_true",
                    help="instead of the bench line: time only the prompt of 2,048 tokens and print one line about it")
    ap.add_argument("--leave-out", action="store_true",
                    help="instead of the bench line: the decode step re-timed with one kind of launch left out at a "
                         "time (its results are then wrong; only its time is of interest), one line per kind")
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
    from trapetum_b200.engine import Engine
    cfg = dict(GEMMA2_2B, num_hidden_layers=args.layers)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    model = build_model(cfg, seed=2)
    V = cfg["vocab_size"]
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    engine = Engine(model, max_tokens=max_batch * args.context, max_slots=max_batch)
    for g in engine.cache.groups:                         # random keys and values, small enough for a sane softmax
        g.k.normal_(0.0, 0.5)
        g.v.normal_(0.0, 0.5)

    if args.leave_out:
        return leave_out_report(engine, model, cfg, torch, args, warmup)
    if args.prefill_only:
        pms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=max(1, args.steps), warmup=warmup)
        print(json.dumps({"prefill_ms": round(pms, 3), "tokens": PREFILL_TOKENS, "layers": args.layers,
                          "frac": round(prefill_flops(cfg, PREFILL_TOKENS) / (pms * 1e-3) / (bf16_tflops * 1e12), 4),
                          "of": peak_src}))
        return 0

    with ClockSampler() as clocks:
        dev_ms, e2e_ms, launches, h2d = time_decode(engine, torch, args.batch, args.context, args.steps, warmup, V)
    value = args.batch * 1e3 / dev_ms
    step_bytes = weight_bytes(cfg) + args.batch * cache_bytes(cfg, args.context - args.steps)
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9

    out = {
        "metric": "decode tok/s at batch %d (Gemma-2-2B)" % args.batch,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights seed 2, uniform token ids, random cache contents)",
        "config": {"model": "gemma-2-2b-shape", "global_batch": args.batch, "seq_len": args.context,
                   "parallelism": "1 gpu", "layers": args.layers, "layers_of_model": GEMMA2_2B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "window": cfg["sliding_window"],
                   "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (each step reads every weight)",
                   "peaks": peak_src},
        "clocks": clocks.summary(),
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4), "of": peak_src, "bytes_per_step": step_bytes},
    }
    if not args.no_points:
        pts = {}
        for b in (1, 64):
            ms, _, _, _ = time_decode(engine, torch, b, args.context, max(8, args.steps // 2), warmup, V)
            pts[f"decode_b{b}"] = round(b * 1e3 / ms, 1)
        out["points"] = pts
        pms = time_prefill(engine, torch, PREFILL_TOKENS, V, reps=5, warmup=3)
        fl = prefill_flops(cfg, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / pms, 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / (bf16_tflops * 1e12), 4), "of": peak_src}
    from trapetum_b200.csrc import ops
    err = ops.kernel_errors()
    if err:
        out["error"] = f"a bounded wait ran out: {err}"
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Command line.

    gemma_run <model_dir> <prompt.bin> [<prompt.bin> ...] [options]
    gemma_run --random-weights <config.json> --seed S --out <model_dir>
    gemma_run --random-weights <config.json> --seed S <prompt.bin> [...] [options]

In the manner of the reference's ``gemma_run <model.cbk> <prompt.bin>``
(runtime/src/bin/gemma_run.rs:2-18): positional model and prompt, the prompt a file
of little-endian int32 token ids as its exporter writes it (model/export_gemma.py:77-78),
greedy continuation of 24 tokens by default, and the same three lines of output
(load time and prompt, continuation ids, ms/token and tok/s).  Several prompt
files run as one batch.  ``--random-weights`` with ``--out`` writes a model folder; without
``--out`` the model of that configuration and seed is made on the device (the same values, no
folder) and the prompts run on it.  The sampling options carry the names of the reference
server's request fields (runtime/src/bin/serve.rs:1284-1292): ``--max_tokens``,
``--temperature``, ``--top_p``, ``--repetition_penalty``.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np


def read_prompt(path: str):
    return np.fromfile(path, dtype="<i4").astype(np.int64).tolist()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gemma_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model", nargs="?", help="model folder (config.json + model.safetensors)")
    ap.add_argument("prompts", nargs="*", help="prompt files: little-endian int32 token ids")
    ap.add_argument("--prompt_ids", action="append", default=[],
                    help="a prompt given as comma-separated ids (may be repeated)")
    ap.add_argument("--max_tokens", "--max-tokens", type=int, default=24)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top_p", "--top-p", type=float, default=0.95)
    ap.add_argument("--repetition_penalty", "--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--stop_id", "--stop-id", type=int, action="append", default=None,
                    help="stop token id (may be repeated; default: the model's eos_token_id)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--host", default=None, choices=["native", "python", "auto"],
                    help="which host runs the model: the native library, this package's own loop, or (default) the "
                         "native one where every part of the model has a native class")
    ap.add_argument("--max_batch", "--max-batch", type=int, default=64)
    ap.add_argument("--random-weights", "--random_weights", metavar="CONFIG_JSON",
                    help="seeded random weights for this config.json: written to --out, or, without --out, made on "
                         "the device for this run")
    ap.add_argument("--out", help="folder that --random-weights writes")
    ap.add_argument("--std", type=float, default=0.02)
    ap.add_argument("--norm_std", "--norm-std", type=float, default=0.1)
    args = ap.parse_args(argv)

    import trapetum_b200 as tb
    if args.random_weights and args.out:
        with open(args.random_weights) as f:
            cfg = json.load(f)
        tb.write_random_model(args.out, cfg, args.seed, args.std, args.norm_std)
        print(f"wrote {args.out} (seed {args.seed})")
        return 0
    if args.random_weights and args.model:
        args.prompts = [args.model] + args.prompts          # no model folder: every positional is a prompt
        args.model = None
    if not args.model and not args.random_weights:
        ap.error("the model folder is missing")
    prompts = [read_prompt(p) for p in args.prompts]
    prompts += [[int(x) for x in s.split(",") if x.strip()] for s in args.prompt_ids]
    if not prompts:
        ap.error("no prompt: give a prompt.bin file or --prompt_ids")

    t0 = time.time()
    if args.random_weights:
        with open(args.random_weights) as f:
            model = tb.random_model(json.load(f), args.seed, args.std, args.norm_std, args.dtype, args.device, host=args.host)
    else:
        model = tb.load_model(args.model, args.dtype, args.device, host=args.host)
    print(f"loaded in {time.time() - t0:.1f}s vocab={model.vocab_size} "
          + " ".join(f"prompt={len(p)} tokens {p}" for p in prompts), flush=True)
    import torch
    torch.cuda.synchronize()
    t0 = time.time()
    outs = tb.generate(model, prompts, max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                       repetition_penalty=args.repetition_penalty, seed=args.seed, stop_ids=args.stop_id,
                       max_batch=args.max_batch)
    torch.cuda.synchronize()
    dt = time.time() - t0
    for o in outs:
        print(f"continuation ids: {o}")
    n = max(1, sum(len(o) for o in outs))
    print(f"decode: {dt * 1e3 / max(1, max(len(o) for o in outs)):.1f} ms/token ({n / dt:.1f} tok/s), "
          f"trapetum_b200 {args.dtype}")
    return 0


if __name__ == "__main__":
    sys.exit(main())

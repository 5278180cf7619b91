#!/usr/bin/env python3
"""Makes tests/golden/safetensors_reader.json.

The whole Gemma-2 model of neuralboot/trapetum cannot run on a CPU (Rust host code over CUDA
kernels), so there are no golden logits.  What does run here is its pure-numpy safetensors
reader, model/export_safetensors.py:24-48 (`_read_safetensors`).  This script writes the Tiny A
model folder (seed 0) with this library's writer, reads it back with the reference's reader and
stores, per tensor, the shape, the float64 sum, the float64 sum of magnitudes and the first four
values.  tests/test_weights.py compares this library's reader with them.

    python tests/golden/make_safetensors_golden.py /path/to/reference
"""
import importlib.util
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))


def main():
    ref_root = sys.argv[1]
    spec = importlib.util.spec_from_file_location("ref_export_safetensors",
                                                  os.path.join(ref_root, "model", "export_safetensors.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.argv = [sys.argv[0]]
    try:
        spec.loader.exec_module(mod)
    except SystemExit:
        pass
    import trapetum_b200 as tb
    from conftest import TINY_A
    with tempfile.TemporaryDirectory() as d:
        tb.write_random_model(d, TINY_A, 0, 0.02, 0.1)
        w = mod._read_safetensors(os.path.join(d, "model.safetensors"))
    out = {}
    for name, a in w.items():
        a = np.asarray(a, dtype=np.float64)
        out[name] = {"shape": list(a.shape), "sum": float(a.sum()), "abs_sum": float(np.abs(a).sum()),
                     "first": [float(x) for x in a.reshape(-1)[:4]]}
    with open(os.path.join(HERE, "safetensors_reader.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(f"{len(out)} tensors")


if __name__ == "__main__":
    main()

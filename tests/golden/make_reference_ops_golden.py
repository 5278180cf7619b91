#!/usr/bin/env python3
"""Makes tests/golden/reference_ops.json: what neuralboot/trapetum's own CUDA operators compute.

The reference's Gemma-2 model is Rust host code and cannot be run here, but the operators it is made of
live in one CUDA file, runtime/cuda/codebook_gemv.cu, which compiles unchanged for sm_100a and exports
them as C functions: op_rmsnorm (:192-202, :836-839), op_rope (:219-230), op_attn with its soft cap
(:240-270, :865-871), op_gelu_mul (:531-537), op_resadd_h (:539-542), dev_argmax (:548-591).  This script
compiles that file as it is (into baseline/_ref/, which is not committed), runs the operators on the small
float16 cases of reference_ops_cases.py on a GPU and stores their outputs.  tests/test_plain.py compares
the plain implementation's functions with them on the CPU; tests/test_gpu_reference_ops.py repeats the
comparison live where the compiled library is present.

    python tests/golden/make_reference_ops_golden.py /path/to/reference        (needs a CUDA device; without
    the path, or $TRAPETUM_REFERENCE, an already compiled baseline/_ref/libcodebook_gemv.so is used)
"""
import ctypes
import json
import os
import subprocess
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
LIB = os.path.join(ROOT, "baseline", "_ref", "libcodebook_gemv.so")


def build(reference_root: str) -> str:
    """Compile the reference's kernel file, unmodified, for sm_100a (works without a GPU)."""
    src = os.path.join(reference_root, "runtime", "cuda", "codebook_gemv.cu")
    if os.path.exists(LIB) and (not os.path.exists(src) or os.path.getmtime(LIB) >= os.path.getmtime(src)):
        return LIB
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "--shared", "-Xcompiler", "-fPIC",
                    "-o", LIB, src], check=True)
    return LIB


def load(path: str = LIB):
    lib = ctypes.CDLL(path)
    lib.dev_argmax.restype = ctypes.c_uint
    for name in ("op_rmsnorm", "op_rope", "op_attn", "op_gelu_mul", "op_resadd_h", "dev_sync"):
        getattr(lib, name).restype = None
    return lib


def run_all(lib):
    """name -> output of the reference's operator on that case, as a CPU float32 tensor (or an int)."""
    from reference_ops_cases import ATTN, inputs
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    ptr = lambda t: P(t.data_ptr())
    c = inputs()
    out = {}
    torch.cuda.synchronize()

    x = c["rmsnorm"]["x"].cuda()
    w1 = (1.0 + c["rmsnorm"]["w"]).float().cuda()                # the exporter stores 1 + w (model/export_gemma.py:25-26)
    y = torch.empty_like(x)
    lib.op_rmsnorm(ptr(x), ptr(w1), ptr(y), I(x.numel()), F(c["rmsnorm"]["eps"]))
    lib.dev_sync()
    out["rmsnorm"] = y.float().cpu()

    for name in ("rope", "rope_far"):
        x = c[name]["x"].cuda().clone()
        nh, hd = x.shape
        inv = (1.0 / (c[name]["theta"] ** (torch.arange(0, hd, 2).float() / hd))).cuda()     # model/export_gemma.py:53
        lib.op_rope(ptr(x), I(c[name]["pos"]), I(nh), I(hd), ptr(inv))
        lib.dev_sync()
        out[name] = x.float().cpu()

    for name, nh, nkv, hd, n, cap in ATTN:
        q, k, v = (c[name][t].cuda().contiguous() for t in ("q", "k", "v"))
        o = torch.empty_like(q)
        lib.op_attn(ptr(q), ptr(k), ptr(v), ptr(o), I(nh), I(nkv), I(hd), I(n), F(cap))
        lib.dev_sync()
        out[name] = o.float().cpu()

    g, u = c["gelu_mul"]["gate"].cuda(), c["gelu_mul"]["up"].cuda()
    y = torch.empty(g.numel(), dtype=torch.float16, device="cuda")
    lib.op_gelu_mul(ptr(g), ptr(u), ptr(y), I(g.numel()))
    lib.dev_sync()
    out["gelu_mul"] = y.float().cpu()

    h, d = c["resadd_h"]["h"].cuda().clone(), c["resadd_h"]["d"].cuda()
    lib.op_resadd_h(ptr(h), ptr(d), I(h.numel()))
    lib.dev_sync()
    out["resadd_h"] = h.float().cpu()

    a = c["argmax"]["logits"].cuda()
    out["argmax"] = int(lib.dev_argmax(ptr(a), I(a.numel())))
    torch.cuda.synchronize()
    return out


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRAPETUM_REFERENCE", "")
    lib = load(build(ref))
    if not torch.cuda.is_available():
        print(f"built {LIB}; run this script again on a machine with a GPU to write the outputs")
        return
    res = run_all(lib)
    stored = {k: (v if isinstance(v, int) else {"shape": list(v.shape), "values": [float(x) for x in v.reshape(-1)]})
              for k, v in res.items()}
    with open(os.path.join(HERE, "reference_ops.json"), "w") as f:
        json.dump({"source": "runtime/cuda/codebook_gemv.cu, compiled unchanged for sm_100a, run on " +
                             torch.cuda.get_device_name(0), "outputs": stored}, f)
    print(f"{len(stored)} cases written")


if __name__ == "__main__":
    main()

"""Random weights from a counter-based generator: element ``i`` of tensor ``name`` is a function of
``(seed, name, i)`` alone.

The same function exists twice in the library: here in numpy, for model folders written on the host,
and in ``csrc/random_init.cu``, which fills tensors in place on the device (a model of 54 GB is never
held in host memory).  Both give the same bits, so a folder and a device-made model of one seed are
the same model.  The reference seeds an xorshift generator inside the program for its synthetic
check models (runtime/src/lib.rs:1604-1629, runtime/src/bin/model.rs:158-177).

Recipe: key = FNV-1a-64(name) xor seed; Philox-4x32-10 on the counter (i // 4, 'TRAP', 0); Box and
Muller's transform on word pairs (0, 1) and (2, 3), with logarithm, sine and cosine as polynomials in
single-precision round-to-nearest arithmetic (no fused operations, so every machine agrees); value =
bfloat16(normal * std).
"""
from __future__ import annotations

from typing import Tuple

import numpy as np
import torch

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_S32 = np.uint64(32)
CHUNK = 1 << 22          # elements made at a time on the host


def name_key(seed: int, name: str) -> Tuple[int, int]:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    h ^= int(seed) & 0xFFFFFFFFFFFFFFFF
    return h & 0xFFFFFFFF, h >> 32


def _philox(blk: np.ndarray, k0: int, k1: int):
    c0, c1 = blk & _MASK, blk >> _S32
    c2 = np.full_like(blk, 0x54524150)
    c3 = np.zeros_like(blk)
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = (p1 >> _S32) ^ c1 ^ np.uint64(k0), p1 & _MASK, (p0 >> _S32) ^ c3 ^ np.uint64(k1), p0 & _MASK
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def _horner(z: np.ndarray, coeffs) -> np.ndarray:
    p = np.full_like(z, np.float32(coeffs[0]))
    for c in coeffs[1:]:
        p = p * z + np.float32(c)
    return p


def _neg_log_unit(w: np.ndarray) -> np.ndarray:
    k = (w >> np.uint64(8)) + np.uint64(1)                     # 1 .. 2^24
    m, e = np.frexp(k.astype(np.float32))                      # k = m * 2^e with m in [0.5, 1)
    m = m * np.float32(2.0)
    e = e - 1
    s = (m - np.float32(1.0)) / (m + np.float32(1.0))
    p = _horner(s * s, (0.0909090936, 0.111111112, 0.142857149, 0.200000003, 0.333333343, 1.0))
    ln_m = np.float32(2.0) * (s * p)
    return (24 - e).astype(np.float32) * np.float32(0.693147182) - ln_m


def _sin_cos_turn(w: np.ndarray):
    q = (w >> np.uint64(30)).astype(np.int64)
    t = ((w >> np.uint64(6)) & np.uint64(0xFFFFFF)).astype(np.float32) * np.float32(2.0 ** -24) * np.float32(1.57079637)
    z = t * t
    s = (_horner(z, (1.60590444e-10, -2.50521079e-08, 2.75573188e-06, -0.000198412701, 0.00833333377,
                     -0.166666672, 1.0))) * t
    c = _horner(z, (2.08767559e-09, -2.755732e-07, 2.48015876e-05, -0.00138888892, 0.0416666679, -0.5, 1.0))
    sn = np.choose(q, [s, c, -s, -c])
    cs = np.choose(q, [c, -s, -c, s])
    return sn, cs


def _round_bf16(v: np.ndarray) -> np.ndarray:
    """float32 -> the float32 that holds the nearest bfloat16 (ties to even)."""
    u = v.view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def normal_host(n: int, key: Tuple[int, int], std: float, first: int = 0) -> np.ndarray:
    """Elements ``first .. first+n`` of the tensor with this key, as float32 that hold bfloat16 values.
    ``first`` must be a multiple of 4."""
    if first % 4:
        raise ValueError("normal_host: 'first' must be a multiple of 4")
    blocks = (n + 3) // 4
    blk = np.arange(first // 4, first // 4 + blocks, dtype=np.uint64)
    c0, c1, c2, c3 = _philox(blk, *key)
    out = np.empty((blocks, 4), dtype=np.float32)
    with np.errstate(over="ignore"):
        for h, (a, b) in enumerate(((c0, c1), (c2, c3))):
            r = np.sqrt(np.float32(2.0) * _neg_log_unit(a))
            sn, cs = _sin_cos_turn(b)
            out[:, 2 * h] = (r * cs) * np.float32(std)
            out[:, 2 * h + 1] = (r * sn) * np.float32(std)
    return _round_bf16(out.reshape(-1)[:n])


def fill_normal(t: torch.Tensor, seed: int, name: str, std: float) -> torch.Tensor:
    """Fill ``t`` (bfloat16 or float32, contiguous) in place with the values of tensor ``name`` for ``seed``:
    on the device by the kernel, on the host by numpy."""
    if not t.is_contiguous() or t.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("fill_normal: wants a contiguous bfloat16 or float32 tensor")
    key = name_key(seed, name)
    if t.is_cuda:
        from ..csrc import ops
        ops.random_normal(t, key, std)
        return t
    flat = t.view(-1)
    for lo in range(0, flat.numel(), CHUNK):
        n = min(CHUNK, flat.numel() - lo)
        flat[lo:lo + n] = torch.from_numpy(normal_host(n, key, std, lo)).to(t.dtype)
    return t

"""Weights by tensor name.

Every part of a model declares the tensors it wants (:class:`TensorSpec`: shape
and role).  :func:`load_tensors` fetches them from a model folder and reports
*all* problems at once: names the file lacks, names nobody asked for, and
shapes that do not fit.  The reference's format is positional and has no such
check (runtime/src/lib.rs:4564-4604: a short or mismatched file ends in a panic
inside ``read_exact``).

Storage rules: tensors stored in bfloat16 are kept so when the engine runs in
bfloat16; a tensor stored in 32 bits stays in 32 bits; integer tables become
int32; the float32 engine up-casts every float tensor to float32 (bfloat16 ->
float32 is exact: the 16 bits become the upper half of the word, as
model/export_safetensors.py:38-40 does on the host).  float16 has three bits
more than bfloat16, so a float16 tensor is never rounded in silence: by default
(``fp16="widen"``) it is widened to float32, which is exact and sends its
products down the 32-bit path; ``fp16="round"`` rounds it to bfloat16 on
request; ``fp16="refuse"`` reports it as a wrong dtype.

:func:`write_random_model` is the random-weights mode: it writes a model folder
(config.json and model.safetensors) from a configuration and a seed.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors_io import WeightFileError, open_model_files, write_safetensors


class WeightError(RuntimeError):
    """Missing, unexpected or wrongly shaped tensors; the message lists them all."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong dtype ({len(self.wrong_kind)}): " + ", ".join(
                f"{n} is {got}, expected {want}" for n, got, want in self.wrong_kind))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one tensor.

    role: ``"matrix"`` and ``"embedding"`` are drawn N(0, std) in random mode,
    ``"norm"`` N(0, norm_std); ``"table"`` is an integer table (zeros in random
    mode).  ``optional`` tensors may be absent (the part then falls back, for
    instance a tied output head)."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


def _is_float(dt: torch.dtype) -> bool:
    return dt in (torch.bfloat16, torch.float16, torch.float32, torch.float64)


FP16_POLICIES = ("widen", "round", "refuse")


def storage_dtype(stored: torch.dtype, role: str, engine_dtype: torch.dtype, fp16: str = "widen") -> torch.dtype:
    """The dtype a tensor has on the device, given how the file stores it."""
    if role == "table":
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32          # stored in 32 bits: stays so
    if stored == torch.float16 and fp16 != "round":
        return torch.float32          # exact; bfloat16 would drop three bits of every value
    return torch.bfloat16


def load_tensors(folder: str, wanted: Dict[str, TensorSpec], engine_dtype: torch.dtype,
                 device, fp16: str = "widen") -> Dict[str, torch.Tensor]:
    if fp16 not in FP16_POLICIES:
        raise ValueError(f"fp16 must be one of {FP16_POLICIES}, got {fp16!r}")
    files = open_model_files(folder)
    missing, unexpected, wrong_shape, wrong_kind = [], [], [], []
    for name, spec in wanted.items():
        if name not in files:
            if not spec.optional:
                missing.append(name)
            continue
        got = files[name].shape(name)
        if tuple(got) != tuple(spec.shape):
            wrong_shape.append((name, got, spec.shape))
        stored = files[name].dtype(name)
        if spec.role == "table" and _is_float(stored):
            wrong_kind.append((name, str(stored).replace("torch.", ""), "an integer type"))
        if spec.role != "table" and not _is_float(stored):
            wrong_kind.append((name, str(stored).replace("torch.", ""), "a floating-point type"))
        if spec.role != "table" and stored == torch.float16 and fp16 == "refuse" and engine_dtype != torch.float32:
            wrong_kind.append((name, "float16", "bfloat16 or float32 (float16 does not fit bfloat16 without rounding; "
                                                "load with fp16='widen' or fp16='round')"))
    for name in files:
        if name not in wanted:
            unexpected.append(name)
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(folder, sorted(missing), sorted(unexpected), wrong_shape, wrong_kind)

    out: Dict[str, torch.Tensor] = {}
    for name, spec in wanted.items():
        if name not in files:
            continue
        f = files[name]
        dt = storage_dtype(f.dtype(name), spec.role, engine_dtype, fp16)
        t = f.tensor(name)
        # .to() copies out of the memory map; the device copy owns its bytes
        out[name] = t.to(device=device, dtype=dt, copy=True).contiguous()
    for f in set(files.values()):
        f.close()
    return out


def random_tensors(wanted: Dict[str, TensorSpec], seed: int, std: float, norm_std: float,
                   dtype: torch.dtype = torch.bfloat16, device="cpu",
                   norm_dtype: Optional[torch.dtype] = None) -> Iterable[Tuple[str, torch.Tensor]]:
    """Seeded random tensors, one at a time, made where they will live (``device``).  Element ``i`` of tensor
    ``name`` depends on ``(seed, name, i)`` only (:mod:`.random_init`), so the order of ``wanted`` does not
    matter and a tensor made on the device equals the one a model folder of the same seed holds.  Values are
    bfloat16 numbers, whatever ``dtype`` stores them in."""
    from .random_init import fill_normal
    for name, spec in wanted.items():
        if spec.optional:
            continue
        if spec.role == "table":
            yield name, torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        dt = norm_dtype if (spec.role == "norm" and norm_dtype is not None) else dtype
        t = torch.empty(spec.shape, dtype=dt, device=device)
        yield name, fill_normal(t, seed, name, norm_std if spec.role == "norm" else std)


def write_random_model(folder: str, config: dict, seed: int, std: float = 0.02, norm_std: float = 0.1,
                       norm_dtype: Optional[torch.dtype] = None, device=None) -> str:
    """Random-weights mode: make ``folder`` a model folder for ``config``.

    The reference's checks build synthetic models from a fixed seed in the same
    spirit (runtime/src/bin/model.rs:158-177).  Values are rounded to bfloat16
    before they are stored, so every reader sees the same numbers.  Tensors are
    made and written one at a time (on ``device``; default: the GPU if there is
    one, it is much faster, else the host; the bits are the same), so the model is
    never held in memory as a whole."""
    from ..engine.model import tensor_specs_for_config  # late: avoids an import cycle
    wanted = tensor_specs_for_config(config)
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=1)
    layout = []
    for name, spec in wanted.items():
        if spec.optional:
            continue
        dt = torch.int32 if spec.role == "table" else \
            (norm_dtype if (spec.role == "norm" and norm_dtype is not None) else torch.bfloat16)
        layout.append((name, dt, tuple(spec.shape)))
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(wanted, seed, std, norm_std, device=device, norm_dtype=norm_dtype),
                      metadata={"format": "pt", "seed": seed}, layout=layout)
    return folder

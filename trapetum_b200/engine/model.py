"""A model put together from a :class:`ModelSpec`, and its loading.

:class:`Model` is the same class for every architecture: it builds the parts the
spec names, collects the tensors they declare, hands the loaded tensors back to
them and runs the schedule.  What differs between architectures is the spec
(``trapetum_b200.models``) and, when needed, new part kinds.

One forward pass (runtime/src/lib.rs:4553-4561 is the reference's, for one token):
embedding -> the schedule's layer calls, each on the residual stream with its
view of the cache -> rows whose logits are wanted -> final norm -> head.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.base import ModelSpec, load_config
from ..csrc import build, ops
from ..parts import ResidualStream, Runtime, build_part
from ..weights.loader import TensorSpec, load_tensors


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec, self.rt = spec, rt
        self.embedding = build_part("embedding", spec.embedding, "", rt)
        self.blocks = []
        for layer in spec.layers:
            mixer = build_part("mixer", layer.mixer, layer.prefix, rt)
            ffn = build_part("feed_forward", layer.feed_forward, layer.prefix, rt)
            self.blocks.append(build_part("block", layer.block, layer.prefix, rt, mixer=mixer, feed_forward=ffn))
        self.final_norm = build_part("norm", spec.final_norm, "", rt)
        self.head = build_part("head", spec.head, "", rt)
        self.vocab_size = spec.vocab_size

    def parts(self):
        return [self.embedding] + self.blocks + [self.final_norm, self.head]

    # -- weights ----------------------------------------------------------------
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for p in self.parts():
            for name, ts in p.tensor_specs().items():
                if name in specs and specs[name].shape != ts.shape:
                    raise ValueError(f"tensor '{name}' is declared with shapes {specs[name].shape} and {ts.shape}")
                # a tensor that one part needs is needed, even if another calls it optional
                if name not in specs or specs[name].optional:
                    specs[name] = ts
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)

    def kernel_files(self) -> Tuple[str, ...]:
        names = ["embed", "sampling"]
        for p in self.parts():
            names.extend(p.kernel_files())
        return tuple(dict.fromkeys(names))

    # -- cache ------------------------------------------------------------------
    def cache_needs(self):
        """(owning entry -> need, owning entry -> entries that read its cache)."""
        needs, readers = {}, {}
        for e, ent in enumerate(self.spec.schedule):
            if ent.cache_of is None:
                needs[e] = self.blocks[ent.layer].mixer.cache_need()
            else:
                readers.setdefault(ent.cache_of, []).append(e)
        return needs, readers

    # -- compute ----------------------------------------------------------------
    def forward(self, ids: torch.Tensor, ctx, cache, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """``ids`` int32 [tokens]; returns float32 logits [wanted rows, vocab]
        (all rows if ``want_rows`` is None)."""
        stream = ResidualStream(self.embedding.forward(ids))
        for e, ent in enumerate(self.spec.schedule):
            owner = e if ent.cache_of is None else ent.cache_of
            self.blocks[ent.layer].forward(stream, ctx, cache.view(e, owner))
        h = stream.value()
        if want_rows is not None:
            h = ops.gather_rows(h, want_rows)
        x = self.final_norm.apply(h, self.rt.dtype)
        return self.head.forward(x)


def tensor_specs_for_config(config: dict) -> Dict[str, TensorSpec]:
    """The tensors a model of this configuration reads, without touching a GPU."""
    _, spec = load_config(config)
    return Model(spec, Runtime(torch.bfloat16, torch.device("cpu"))).tensor_specs()


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"unknown dtype '{dtype}' (bfloat16 or float32)") from None


def load_model(folder: str, dtype="bfloat16", device="cuda:0", fp16: str = "widen") -> Model:
    """Read config.json, pick the model by its architecture name, load and bind the weights.
    ``fp16``: what happens to tensors stored in float16 when the engine computes in bfloat16: "widen" keeps
    them exactly, as float32 (their products then take the 32-bit path), "round" rounds them to bfloat16,
    "refuse" reports them (see :mod:`trapetum_b200.weights.loader`)."""
    import trapetum_b200.models  # noqa: F401  (registers the architectures)
    dt = parse_dtype(dtype)
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("trapetum_b200 computes on a CUDA device only (no CPU path); got device " + str(device))
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is visible; trapetum_b200 has no CPU path")
    _, spec = load_config(folder)
    model = Model(spec, Runtime(dt, dev))
    build.require(model.kernel_files())
    tensors = load_tensors(folder, model.tensor_specs(), dt, dev, fp16)
    model.bind(tensors)
    return model


def random_model(config, seed: int = 0, std: float = 0.02, norm_std: float = 0.1, dtype="bfloat16",
                 device="cuda:0") -> Model:
    """A model of ``config`` (a dict of config.json keys, or a path) whose weights are made on the device:
    the same values that ``write_random_model(folder, config, seed, std, norm_std)`` stores, without the
    folder and without a host copy (each tensor is filled in place by the counter-based generator, so a model
    of any size that fits the GPU can be made).  The reference builds the synthetic models of its checks
    inside the program as well (runtime/src/lib.rs:1604-1629)."""
    import trapetum_b200.models  # noqa: F401  (registers the architectures)
    from ..weights.loader import random_tensors
    dt = parse_dtype(dtype)
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("trapetum_b200 computes on a CUDA device only (no CPU path); got device " + str(device))
    _, spec = load_config(config)
    model = Model(spec, Runtime(dt, dev))
    build.require(model.kernel_files() + ("random_init",))
    with torch.cuda.device(dev):
        model.bind(dict(random_tensors(model.tensor_specs(), seed, std, norm_std, dtype=dt, device=dev)))
    return model

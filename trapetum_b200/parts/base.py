"""What a part of a layer is, and the registries that build parts from specs.

A *part* is built from a :class:`PartSpec` (kind + parameters) and a
:class:`Runtime` (compute dtype and device).  It says which tensors it needs
(:meth:`Part.tensor_specs`), receives them (:meth:`Part.bind`) and then
computes.  Five kinds of part exist, each with its own registry and interface:

=================  ==========================================================
norm               ``apply(x, out_dtype) -> y``; may offer fused forms with the
                   residual sum (:class:`Norm`)
position           position encoding used by a mixer (:class:`PositionEncoding`)
mixer              token mixing with a cache (:class:`Mixer`): attention here
feed_forward       per-token transform (:class:`FeedForward`): dense or experts
block              the arrangement of a layer's parts around the residual
                   stream (:class:`Block`)
=================  ==========================================================

plus ``embedding`` and ``head`` at the two ends of the model.  No part knows
which model it is in: sizes, constants and tensor names all arrive as
parameters.  Registering a new kind needs no change to this package::

    from trapetum_b200.parts import register_part
    register_part("mixer", "my_mixer", MyMixer)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from ..config.base import ConfigError, PartSpec
from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class Runtime:
    """How the model computes: the activations' dtype and the device."""
    dtype: torch.dtype            # torch.bfloat16 or torch.float32
    device: torch.device


# ---------------------------------------------------------------------------
# What a mixer may ask of the cache
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class KVNeed:
    """Keys and values per token.  ``window`` None: all of them are kept;
    an integer: only the last ``window`` tokens are ever read."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size: ``shape`` numbers of ``dtype`` (float32 unless
    said otherwise; any torch dtype), zeroed when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ---------------------------------------------------------------------------
# Interfaces
# ---------------------------------------------------------------------------

class Part:
    """Base of all parts."""

    def __init__(self, params: Dict[str, Any], prefix: str, rt: Runtime):
        self.params = params
        self.prefix = prefix
        self.rt = rt

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Full tensor names -> what is expected of them."""
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the loaded tensors (a dict that holds at least the declared names)."""

    def kernel_files(self) -> Tuple[str, ...]:
        """Kernel libraries this part launches, so that they can be built together."""
        return ()

    def _name(self, key: str) -> str:
        return self.prefix + self.params[key]


class Norm(Part):
    def apply(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError

    def add_to(self, h: torch.Tensor, a: torch.Tensor, then: Optional["Norm"], out_dtype) -> Optional[torch.Tensor]:
        """``h += self(a)`` in place; if ``then`` is given, also return ``then(h)``.
        The default composes the two; a norm may fuse them."""
        from ..csrc import ops
        if a.dim() == 3:                              # split-K partial sums: add them up first
            a = ops.sum_partials(a.contiguous())
        ops.residual_add(h, self.apply(a.contiguous(), torch.float32))
        return then.apply(h, out_dtype) if then is not None else None


class PositionEncoding(Part):
    def rotary_table(self):
        """``(inv_freq, rotary_dim)`` if this encoding is the rotate-half rotation of the first ``rotary_dim`` dims
        of q and k by ``position * inv_freq[i]`` (``(None, 0)``: it changes nothing), so that a mixer's kernel
        may apply it itself; None if it is anything else (the mixer then calls ``rotate_and_store``)."""
        return None


class Mixer(Part):
    def cache_need(self):
        """:class:`KVNeed`, :class:`StateNeed` or None."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        """``x`` [tokens, hidden] in the compute dtype; ``ctx`` the step's
        :class:`~trapetum_b200.engine.step.StepContext`; ``cache`` this call's view
        of the cache (:class:`~trapetum_b200.cache.kv.KVLineView`, a state tensor
        view, or None).  Returns [tokens, hidden], or [splits, tokens, hidden] float32 partial
        sums whose sum over the first axis is the result (the residual stream adds them)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arranges a mixer and a feed-forward around the residual stream."""

    def __init__(self, params, prefix, rt, mixer: Mixer, feed_forward: FeedForward):
        super().__init__(params, prefix, rt)
        self.mixer = mixer
        self.feed_forward = feed_forward

    def forward(self, stream, ctx, cache) -> None:
        raise NotImplementedError


# ---------------------------------------------------------------------------
# Registries
# ---------------------------------------------------------------------------

_KINDS = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, Callable]] = {k: {} for k in _KINDS}


def register_part(family: str, kind: str, cls) -> None:
    if family not in _REGISTRY:
        raise ValueError(f"unknown part family '{family}' (families: {', '.join(_KINDS)})")
    _REGISTRY[family][kind] = cls


def build_part(family: str, spec: PartSpec, prefix: str, rt: Runtime, **extra):
    try:
        cls = _REGISTRY[family][spec.kind]
    except KeyError:
        raise ConfigError(f"no {family} of kind '{spec.kind}' is registered "
                          f"(known: {', '.join(sorted(_REGISTRY[family])) or 'none'})") from None
    return cls(spec.params, prefix, rt, **extra)


def known_parts(family: str):
    return sorted(_REGISTRY[family])

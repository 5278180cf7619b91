"""The residual stream of a step: a 32-bit [tokens, hidden] matrix and the one
branch output that still waits to be added.

Blocks never add into the stream themselves.  They call :meth:`add` or
:meth:`add_normed` with a branch output and :meth:`normed` when they need the
next normalised input; the stream holds an addition back until the next read
so that ``h += norm_a(a); x = norm_b(h)`` runs as one kernel, also across the
border between two layers.  The sum itself is always 32-bit.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import Norm


class ResidualStream:
    def __init__(self, h: torch.Tensor):
        assert h.dtype == torch.float32
        self.h = h
        self._pending = None          # (branch output, its norm or None)

    def add(self, a: torch.Tensor) -> None:
        """h += a (no norm on the branch output)."""
        self._flush()
        self._pending = (a, None)

    def add_normed(self, a: torch.Tensor, norm: Norm) -> None:
        """h += norm(a)."""
        self._flush()
        self._pending = (a, norm)

    def normed(self, norm: Norm, out_dtype: torch.dtype) -> torch.Tensor:
        """norm(h), after whatever addition was still waiting."""
        if self._pending is not None:
            a, post = self._pending
            self._pending = None
            if post is not None:
                return post.add_to(self.h, a, norm, out_dtype)
            ops.residual_add(self.h, a)
        return norm.apply(self.h, out_dtype)

    def value(self) -> torch.Tensor:
        self._flush()
        return self.h

    def _flush(self) -> None:
        if self._pending is None:
            return
        a, post = self._pending
        self._pending = None
        if post is not None:
            post.add_to(self.h, a, None, None)
        else:
            ops.residual_add(self.h, a)

"""Rotary position encoding (rotate-half pairing).

For each head and i in [0, R/2): ``angle = pos * theta^(-2i/R)`` and the pair
``(x[i], x[i+R/2])`` is rotated by it (runtime/cuda/codebook_gemv.cu:219-230;
the table of inverse frequencies is made as in model/export_gemma.py:53).  R is
``rotary_dim`` (the whole head for Gemma-2).  The table is made once, in
32-bit; the kernel multiplies by the position and takes sin and cos in 32-bit.
The rotation is fused with the cache write, so a mixer hands this part its qkv
matrix and its cache line in one call.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import PositionEncoding, register_part


class Rope(PositionEncoding):
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= self.head_dim):
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        self._inv_freq_cpu = 1.0 / (torch.tensor(self.theta, dtype=torch.float32) ** (idx / self.rotary_dim))
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, tensors) -> None:
        self.inv_freq = self._inv_freq_cpu.to(self.rt.device)

    def kernel_files(self):
        return ("rope_kv",)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim

    def rotate_and_store(self, qkv, n_heads, n_kv_heads, ctx, line, store: bool, partial=None) -> None:
        """Rotate q and k inside ``qkv`` at the step's positions; with ``store`` also
        write k and v into the cache line.  ``partial``: split-K partial sums of the projection
        ([splits, tokens, width] float32) to take the values from; ``qkv`` is then only written."""
        ops.rope_kv(qkv, n_heads, n_kv_heads, self.head_dim, self.rotary_dim, self.inv_freq,
                    ctx.positions, ctx.token_seq, ctx.len_after,
                    line.k if store else None, line.v if store else None,
                    line.page_table if store else None, line.ring_rows if store else 0, partial)


class NoPosition(PositionEncoding):
    """No position encoding: keys and values are stored as they are."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.head_dim = int(params["head_dim"])

    def kernel_files(self):
        return ("rope_kv",)

    def rotary_table(self):
        return None, 0

    def rotate_and_store(self, qkv, n_heads, n_kv_heads, ctx, line, store: bool, partial=None) -> None:
        if store or partial is not None:
            ops.rope_kv(qkv, n_heads, n_kv_heads, self.head_dim, 0, None, ctx.positions, ctx.token_seq,
                        ctx.len_after, line.k if store else None, line.v if store else None,
                        line.page_table if store else None, line.ring_rows if store else 0, partial)


register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)

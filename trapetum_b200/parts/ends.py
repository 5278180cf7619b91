"""The two ends of a model: token embedding and output head.

Embedding: ``h[t] = E[id_t] * scale`` into the 32-bit residual stream; Gemma-2's
scale is sqrt(hidden) (model/export_gemma.py:59-61).  Head: ``logits = x W^T``
in 32-bit, then ``cap * tanh(logits / cap)`` if a cap is set
(runtime/src/lib.rs:4557-4560, where the cap runs on the host); W is the
embedding table itself when the head is tied (model/export_gemma.py:73 writes
the tied weight unscaled) unless the file brings a matrix under the head's own name.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Part, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear


class Embedding(Part):
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self._name("weight"): TensorSpec((self.vocab, self.hidden), "embedding")}

    def bind(self, tensors) -> None:
        self.table = tensors[self._name("weight")]

    def kernel_files(self):
        return ("embed",)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embed(ids, self.table, self.scale)


class LinearHead(Part):
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.softcap = float(params["softcap"]) if params.get("softcap") else 0.0
        self.tied_to = params.get("tied_to")
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self._name("weight"): TensorSpec((self.vocab, self.hidden), "matrix", optional=bool(self.tied_to))}
        if self.tied_to:
            specs[self.prefix + self.tied_to] = TensorSpec((self.vocab, self.hidden), "embedding")
        return specs

    def bind(self, tensors) -> None:
        own = tensors.get(self._name("weight"))
        self.weight = own if own is not None else tensors[self.prefix + self.tied_to]

    def kernel_files(self):
        return linear_kernels(self.rt.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, torch.float32, self.softcap)


register_part("embedding", "embedding", Embedding)
register_part("head", "linear_head", LinearHead)

"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * (offset + w)``.

``unit_offset`` selects the ``(1 + w)`` form.  The reference adds the 1 to the
stored weights at export (model/export_gemma.py:25-26) and then runs the plain
form (runtime/cuda/codebook_gemv.cu:192-202); here the raw weight is kept and
the sum is made in the kernel in 32-bit.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = 1.0 if params.get("unit_offset") else 0.0
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self._name("weight"): TensorSpec((self.size,), "norm")}

    def bind(self, tensors) -> None:
        self.weight = tensors[self._name("weight")]

    def kernel_files(self):
        return ("norm",)

    def apply(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.offset, out_dtype)

    def add_to(self, h, a, then, out_dtype):
        if then is None:
            return ops.add_rmsnorm(h, a, self.weight, self.eps, self.offset)
        if isinstance(then, RMSNorm) and then.weight.dtype == self.weight.dtype:
            return ops.add_rmsnorm(h, a, self.weight, self.eps, self.offset,
                                   then.weight, then.eps, then.offset, out_dtype)
        ops.add_rmsnorm(h, a, self.weight, self.eps, self.offset)
        return then.apply(h, out_dtype)


register_part("norm", "rmsnorm", RMSNorm)

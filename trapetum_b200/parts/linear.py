"""Matrix product with a weight matrix: the one place that picks a GEMM kernel.

``y[T, N] = x[T, K] @ W[N, K]^T`` with W as the checkpoint stores it ([out, in]).
bfloat16 operands go to the tensor-core kernel when it takes the sizes;
everything else (the 32-bit path, 32-bit weights, odd sizes) goes to the
32-bit FMA kernel.  Accumulation is 32-bit in both.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, softcap: Optional[float] = None) -> torch.Tensor:
    cap = float(softcap) if softcap else 0.0
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ops.gemm_tc_takes(x, w):
        return ops.gemm_tc(x, w, out_dtype, cap)
    return ops.gemm_simt(x, w, out_dtype, cap)


def linear_partials(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """The product as 32-bit partial sums [splits, T, N] (splits may be 1): for outputs that go straight into
    a kernel that reads them once (the residual sum with its norm), which then adds the splits itself."""
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ops.gemm_tc_takes(x, w):
        return ops.gemm_tc(x, w, torch.float32, partials=True)
    return ops.gemm_simt(x, w, torch.float32)[None]


def kernel_files(dtype: torch.dtype):
    from ..csrc import build
    if dtype == torch.bfloat16 and "gemm_tc" in build.SOURCES:
        return ("gemm_simt", "gemm_tc")
    return ("gemm_simt",)

"""Gated dense feed-forward: ``down(act(gate(x)) * up(x))``.

Gemma-2's form is GeGLU with the tanh approximation of GELU
(runtime/src/lib.rs:4511-4516; runtime/cuda/codebook_gemv.cu:531-537); the
activation is a parameter, as are both widths and the three tensor names.  The
gate and up matrices are fused into one when the weights are bound.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear, linear_partials


class GatedMLP(FeedForward):
    graph_safe = True          # every launch depends on device data only
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = params["activation"]
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"gated_mlp: unknown activation '{self.activation}' (known: {sorted(ops.ACTIVATIONS)})")
        self.w_gu: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            self._name("gate"): TensorSpec((self.inter, self.hidden)),
            self._name("up"): TensorSpec((self.inter, self.hidden)),
            self._name("down"): TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors) -> None:
        g, u = tensors[self._name("gate")], tensors[self._name("up")]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        # With bfloat16 weights of tensor-core sizes the activation runs in the product's epilogue; the gate
        # and up rows are then interleaved in blocks of 16.  Otherwise: [gate; up] and a kernel of its own.
        self.fused = (dt == torch.bfloat16 and self.rt.dtype == torch.bfloat16 and self.inter % 16 == 0
                      and self.hidden % 8 == 0)
        if self.fused:
            self.w_gu = ops.interleave_gate_up(g, u)
        else:
            self.w_gu = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = tensors[self._name("down")]

    def kernel_files(self):
        return linear_kernels(self.rt.dtype) + ("activation",)

    def forward(self, x, ctx):
        if self.fused and ops.gemm_tc_takes(x, self.w_gu):
            act = ops.gemm_tc(x, self.w_gu, self.rt.dtype, gated_act=self.activation)
            return linear_partials(act, self.w_down)
        if self.fused:
            raise RuntimeError("gated_mlp: the interleaved weights need the tensor-core product, which does not take "
                               f"an input of shape {tuple(x.shape)} with strides {x.stride()}")
        gu = linear(x, self.w_gu, self.rt.dtype)
        act = ops.gated_act(gu, self.activation, self.rt.dtype)
        return linear_partials(act, self.w_down)


register_part("feed_forward", "gated_mlp", GatedMLP)

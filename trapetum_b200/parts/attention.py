"""Attention as a mixer: grouped-query, causal, optionally windowed and soft-capped.

In the order the reference computes it (runtime/src/lib.rs:4483-4496):
q, k, v projections without bias; position encoding of q and k; k and v appended
to the cache; per query ``s = (q.k) * scale``, ``s = cap * tanh(s / cap)`` if a
cap is set, softmax over the visible keys, weighted sum of v
(runtime/cuda/codebook_gemv.cu:240-270); output projection.  Query head ``h``
reads kv head ``h // (num_heads // num_kv_heads)`` (codebook_gemv.cu:244).

Parameters (none is fixed in code): ``hidden_size``, ``num_heads``,
``num_kv_heads``, ``head_dim``, ``scale``, ``softcap`` (None: off), ``window``
(None: every earlier token is visible; W: the last W tokens, the query's own
included), ``position`` (a position-encoding spec) and the four tensor names.
Optional, absent in Gemma-2: ``bias`` (tensor names of biases under the keys
``q``, ``k``, ``v``, ``o``; any subset) and ``q_norm`` / ``k_norm`` (norm specs
applied to every query / key head, over ``head_dim``, before the position
encoding).  What the fused decode kernel can do by itself is declared by
:meth:`Attention.fused_decode`: the plain projection followed by a rotate-half
rotation.  With a bias or a head norm the same steps run as kernels of their
own, so such a mixer is a matter of parameters, not of a change to a kernel.
The reference fixes ``scale = rsqrt(head_dim)`` (codebook_gemv.cu:250) and has
no window (runtime/src/lib.rs:4455).

The three projections are fused into one matrix when the weights are bound, so
a step runs one product for q, k and v.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, build_part, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear, linear_partials


class Attention(Mixer):
    graph_safe = True          # every launch depends on device data only
    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.window = int(p["window"]) if p.get("window") else None
        if self.n_heads % self.n_kv:
            raise ValueError(f"attention: {self.n_heads} heads cannot share {self.n_kv} kv heads")
        self.position = build_part("position", p["position"], prefix, rt)
        self.qd = self.n_heads * self.hd
        self.kvd = self.n_kv * self.hd
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.bias_names = dict(p.get("bias") or {})
        unknown = set(self.bias_names) - {"q", "k", "v", "o"}
        if unknown:
            raise ValueError(f"attention: 'bias' names {sorted(unknown)}; it knows q, k, v and o")
        self.q_norm = build_part("norm", p["q_norm"], prefix, rt) if p.get("q_norm") else None
        self.k_norm = build_part("norm", p["k_norm"], prefix, rt) if p.get("k_norm") else None
        self.b_qkv: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {
            self._name("q"): TensorSpec((self.qd, self.hidden)),
            self._name("k"): TensorSpec((self.kvd, self.hidden)),
            self._name("v"): TensorSpec((self.kvd, self.hidden)),
            self._name("o"): TensorSpec((self.hidden, self.qd)),
        }
        sizes = {"q": self.qd, "k": self.kvd, "v": self.kvd, "o": self.hidden}
        for key, name in self.bias_names.items():
            specs[self.prefix + name] = TensorSpec((sizes[key],))
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                specs.update(n.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        q, k, v = (tensors[self._name(n)] for n in ("q", "k", "v"))
        dt = q.dtype if (q.dtype == k.dtype == v.dtype) else torch.float32
        self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = tensors[self._name("o")]
        self.position.bind(tensors)
        if any(key in self.bias_names for key in "qkv"):
            # one bias row for the fused projection, 32-bit; a projection without a bias of its own gets zeros
            parts = [tensors[self.prefix + self.bias_names[key]].float() if key in self.bias_names
                     else torch.zeros(n, dtype=torch.float32, device=q.device)
                     for key, n in (("q", self.qd), ("k", self.kvd), ("v", self.kvd))]
            self.b_qkv = torch.cat(parts).contiguous()
        if "o" in self.bias_names:
            self.b_o = tensors[self.prefix + self.bias_names["o"]].float().contiguous()
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                n.bind(tensors)

    def fused_decode(self) -> bool:
        """Whether this mixer is what the decode kernel's own prologue computes: the plain q/k/v projection
        (no bias, no head norm), then a rotate-half rotation (or none)."""
        return self.b_qkv is None and self.q_norm is None and self.k_norm is None \
            and self.position.rotary_table() is not None

    def _finish_projection(self, qkv: torch.Tensor, n_q: int, n_kv: int) -> None:
        """Bias and head norms on a freshly projected [tokens, (n_q + 2 n_kv) * head_dim] matrix, in place."""
        if self.b_qkv is not None:
            ops.add_bias(qkv, self.b_qkv[:qkv.shape[1]])
        T = qkv.shape[0]
        for norm, lo, n in ((self.q_norm, 0, n_q), (self.k_norm, n_q * self.hd, n_kv)):
            if norm is not None and n:
                heads = qkv[:, lo:lo + n * self.hd]
                normed = norm.apply(heads.reshape(T * n, self.hd).contiguous(), qkv.dtype)
                heads.copy_(normed.view(T, n * self.hd))

    def _out(self, o: torch.Tensor) -> torch.Tensor:
        part = linear_partials(o, self.w_o)
        if self.b_o is not None:
            ops.add_bias(part[0], self.b_o)
        return part

    def kernel_files(self):
        fast = ("attention_decode",) if ops.attn_decode_takes(self.rt.dtype, self.n_heads, self.n_kv, self.hd) else ()
        if self.bias_names:
            fast += ("activation",)
        for n in (self.q_norm, self.k_norm):
            if n is not None:
                fast += tuple(n.kernel_files())
        if ops.attn_prefill_tc_takes(self.rt.dtype, self.hd):
            fast += (ops.attn_prefill_tc_lib(self.hd),)
        elif ops.attn_prefill_takes(self.rt.dtype, self.hd):
            fast += (ops.attn_prefill_lib(self.hd),)
        return linear_kernels(self.rt.dtype) + self.position.kernel_files() + ("attention_simt",) + fast

    def cache_need(self):
        return KVNeed(self.n_kv, self.hd, self.window)

    def forward(self, x, ctx, line):
        dt = self.rt.dtype
        if line.owner:
            plain = self.b_qkv is None and self.q_norm is None and self.k_norm is None
            if plain and dt == torch.bfloat16 and x.shape[0] <= 128 and ops.gemm_tc_takes(x, self.w_qkv):
                # few tokens: the product comes as split-K partial sums, which the rotation kernel adds up
                part = ops.gemm_tc(x, self.w_qkv, torch.float32, partials=True)
                rotate = self.position.rotary_table()
                if not ctx.is_prefill and self.fused_decode() and ops.attn_decode_rotates(dt, self.n_heads, self.n_kv, self.hd):
                    # decoding: the attention kernel adds them up, rotates and appends to the cache by itself
                    o = ops.attn_decode(part, line.k, line.v, line.page_table, ctx.len_after, self.n_heads, self.n_kv,
                                        self.hd, self.scale, self.softcap, self.window or 0, line.ring_rows,
                                        ctx.len_bucket, ctx.uneven, rotate)
                    return self._out(o)
                qkv = torch.empty(part.shape[1:], dtype=dt, device=x.device)
                self.position.rotate_and_store(qkv, self.n_heads, self.n_kv, ctx, line, store=True, partial=part)
            else:
                qkv = linear(x, self.w_qkv, dt)
                self._finish_projection(qkv, self.n_heads, self.n_kv)
                self.position.rotate_and_store(qkv, self.n_heads, self.n_kv, ctx, line, store=True)
            q = qkv[:, :self.qd]
            k = qkv[:, self.qd:self.qd + self.kvd]
            v = qkv[:, self.qd + self.kvd:]
            if ctx.is_prefill and line.shared:
                ctx.step_kv[line.entry] = (k, v)      # a later call that reads this cache needs them
        else:
            # this call reads another call's cache: only its queries are new
            q = linear(x, self.w_qkv[:self.qd], dt)
            self._finish_projection(q, self.n_heads, 0)
            self.position.rotate_and_store(q, self.n_heads, 0, ctx, line, store=False)
            k, v = ctx.step_kv[line.entry] if ctx.is_prefill else (None, None)
        if ctx.is_prefill:
            o = ops.attn_prefill(q, k, v, ctx.seq_start, ctx.token_seq, self.n_heads, self.n_kv, self.hd,
                                 self.scale, self.softcap, self.window or 0, ctx.max_seq_len, ctx.seq_lens, ctx.memo)
        else:
            o = ops.attn_decode(q, line.k, line.v, line.page_table, ctx.len_after, self.n_heads, self.n_kv,
                                self.hd, self.scale, self.softcap, self.window or 0, line.ring_rows, ctx.len_bucket,
                                ctx.uneven)
        return self._out(o)


register_part("mixer", "attention", Attention)

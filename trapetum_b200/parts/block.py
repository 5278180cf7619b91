"""Arrangements of a layer's parts around the residual stream.

``sandwich``: a norm before and a norm after each of the two branches
(runtime/src/lib.rs:4527-4540):

    h += post_mixer_norm(mixer(pre_mixer_norm(h)))
    h += post_ffn_norm(feed_forward(pre_ffn_norm(h)))

``pre_norm``: the common two-norm arrangement, branch outputs added as they are:

    h += mixer(pre_mixer_norm(h));  h += feed_forward(pre_ffn_norm(h))

A block only talks to the :class:`~trapetum_b200.parts.stream.ResidualStream`,
which decides how additions and norms are fused.
"""
from __future__ import annotations

from typing import Dict

from ..weights.loader import TensorSpec
from .base import Block, build_part, register_part


class _NormedBlock(Block):
    graph_safe = True          # every launch depends on device data only
    NORMS = ()

    def __init__(self, params, prefix, rt, mixer, feed_forward):
        super().__init__(params, prefix, rt, mixer, feed_forward)
        self.norms = {n: build_part("norm", params[n], prefix, rt) for n in self.NORMS}

    def parts(self):
        return list(self.norms.values()) + [self.mixer, self.feed_forward]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for p in self.parts():
            specs.update(p.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        for p in self.parts():
            p.bind(tensors)

    def kernel_files(self):
        out = ()
        for p in self.parts():
            out += tuple(p.kernel_files())
        return out


class SandwichBlock(_NormedBlock):
    NORMS = ("pre_mixer_norm", "post_mixer_norm", "pre_ffn_norm", "post_ffn_norm")

    def forward(self, stream, ctx, cache) -> None:
        dt = self.rt.dtype
        x = stream.normed(self.norms["pre_mixer_norm"], dt)
        stream.add_normed(self.mixer.forward(x, ctx, cache), self.norms["post_mixer_norm"])
        x = stream.normed(self.norms["pre_ffn_norm"], dt)
        stream.add_normed(self.feed_forward.forward(x, ctx), self.norms["post_ffn_norm"])


class PreNormBlock(_NormedBlock):
    NORMS = ("pre_mixer_norm", "pre_ffn_norm")

    def forward(self, stream, ctx, cache) -> None:
        dt = self.rt.dtype
        x = stream.normed(self.norms["pre_mixer_norm"], dt)
        stream.add(self.mixer.forward(x, ctx, cache))
        x = stream.normed(self.norms["pre_ffn_norm"], dt)
        stream.add(self.feed_forward.forward(x, ctx))


register_part("block", "sandwich", SandwichBlock)
register_part("block", "pre_norm", PreNormBlock)

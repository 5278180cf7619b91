"""Sampling options, named and meant as the reference's server names and means them
(runtime/src/bin/serve.rs:1284-1292): ``temperature`` (<= 0: greedy, the default),
``top_p`` (default 0.95), ``repetition_penalty`` (> 1 penalises the last 128 tokens;
the reference's Gemma command line applies none, runtime/src/bin/gemma_run.rs:13-15,
so the default here is 1.0, its server's default is 1.3) and ``max_tokens`` (default 256).
``seed`` is ours: the reference seeds its generator from the wall clock
(serve.rs:309-311), so its samples cannot be repeated.
"""
from __future__ import annotations

from dataclasses import dataclass

REPETITION_WINDOW = 128          # recent tokens that the penalty looks at (serve.rs:327)

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 0.95
    repetition_penalty: float = 1.0
    max_tokens: int = 256
    seed: int = 0

    def __post_init__(self):
        if self.max_tokens < 0:
            raise ValueError(f"max_tokens must not be negative, got {self.max_tokens}")
        if not (0.0 < self.top_p):
            raise ValueError(f"top_p must be positive, got {self.top_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be positive, got {self.repetition_penalty}")

    @property
    def greedy(self) -> bool:
        return not (self.temperature > 0.0)

    @property
    def needs_sampler(self) -> bool:
        """False when a plain argmax over the logits is the whole job."""
        return (not self.greedy) or self.repetition_penalty > 1.0


def _mix(x: int) -> int:
    """splitmix64 finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def draw_uniform(seed: int, request: int, index: int) -> float:
    """The draw u in [0, 1) for token ``index`` of request ``request``: a counter-based
    generator, so a request's samples do not depend on which batch it ran in."""
    x = _mix(seed & _MASK)
    x = _mix(x ^ ((request + 1) & _MASK))
    x = _mix(x ^ ((index + 1) * 0xD6E8FEB86659FD93 & _MASK))
    return (x >> 40) / float(1 << 24)        # 24 bits: exactly representable in float32

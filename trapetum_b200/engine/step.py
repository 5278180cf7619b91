"""The step function: one batch of sequences, one forward pass.

A batch is a set of sequences that start together.  Its first step brings every
sequence's whole prompt (lengths may differ; tokens are packed back to back, no
padding exists anywhere); every later step brings exactly one token for each
sequence that is still alive.  A step runs only the tokens it is given, on top
of the cache the earlier steps left, and returns the logits at the places asked
for.  The reference's forward takes one token of one sequence and returns all
its logits (runtime/src/lib.rs:4553-4561), so a prompt costs one call per token
(runtime/src/bin/gemma_run.rs:12).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import Cache


class StepError(ValueError):
    """The step's entries do not form a valid step."""


@dataclass
class StepContext:
    """What the parts may know about the running step (all index tensors int32 on the device)."""
    is_prefill: bool
    n_tokens: int
    batch: int
    positions: torch.Tensor          # [tokens] position of each token in its sequence
    token_seq: torch.Tensor          # [tokens] index of each token's sequence in the batch
    seq_start: torch.Tensor          # [batch + 1] first row of each sequence in the packed tokens
    len_after: torch.Tensor          # [batch] tokens of each sequence once this step is done
    slot_ids: torch.Tensor           # [batch] cache slot of each sequence
    slots: List[int]
    seq_lens: List[int]              # tokens this step brings, per sequence (host)
    max_seq_len: int                 # the longest of them
    max_len_after: int
    len_bucket: int = 0              # a power of two >= max_len_after: what launch shapes may depend on
    uneven: int = 0                  # decode: how much the contexts differ in length, 0..3 (launch shapes may depend on it)
    step_kv: Dict[int, tuple] = field(default_factory=dict)   # prefill: entry -> (k, v) of this step
    memo: Dict[str, object] = field(default_factory=dict)     # small per-step values that kernels share across layers


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepInputs:
    """Packs a step's integer inputs into one host buffer, copies it to the device in one
    transfer and hands out views."""

    def __init__(self, device):
        self.device = device
        self._host: Optional[torch.Tensor] = None
        self._dev: Optional[torch.Tensor] = None
        self._copied = None           # event after the last copy: the host buffer is free again

    def upload(self, arrays: Dict[str, np.ndarray]) -> Dict[str, torch.Tensor]:
        offs, total = {}, 0
        for name, a in arrays.items():
            offs[name] = total
            total += _align4(max(a.size, 1))
        if self._host is None or self._host.numel() < total:
            cap = max(1024, 1 << (total - 1).bit_length())
            self._host = torch.empty(cap, dtype=torch.int32).pin_memory() if self.device.type == "cuda" \
                else torch.empty(cap, dtype=torch.int32)
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        if self._copied is not None:
            self._copied.synchronize()
        hv = self._host.numpy()
        for name, a in arrays.items():
            hv[offs[name]:offs[name] + a.size] = a.reshape(-1)
        self._dev[:total].copy_(self._host[:total], non_blocking=True)
        if self.device.type == "cuda":
            self._copied = torch.cuda.Event()
            self._copied.record()
        out = {}
        for name, a in arrays.items():
            out[name] = self._dev[offs[name]:offs[name] + a.size].view(a.shape)
        return out


def classify(cache: Cache, slots: Sequence[int], tokens: Sequence[Sequence[int]]) -> bool:
    """True for a first step (every sequence starts), False for a one-token step; anything else is refused."""
    if len(slots) == 0:
        raise StepError("a step needs at least one sequence")
    if len(set(slots)) != len(slots):
        raise StepError(f"a slot appears twice in one step: {list(slots)}")
    if len(tokens) != len(slots):
        raise StepError(f"{len(slots)} slots but {len(tokens)} token lists")
    lens = [cache.length(s) for s in slots]
    if any(len(t) == 0 for t in tokens):
        raise StepError("every sequence of a step brings at least one token")
    if all(l == 0 for l in lens):
        return True
    if all(l > 0 for l in lens) and all(len(t) == 1 for t in tokens):
        return False
    raise StepError("the sequences of a step either all start (empty cache, whole prompts) or all go on by "
                    f"exactly one token; got cache lengths {lens} and token counts {[len(t) for t in tokens]}")

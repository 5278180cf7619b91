"""The engine: a model, its cache, and the step function over both.

:class:`Engine` is what generation, trace replay and the benchmark all drive;
there is no second forward pass anywhere.

    engine = Engine(model, max_tokens=4096)
    slots = engine.start(3)                         # three sequences that start together
    logits = engine.step(slots, prompts, want)      # whole prompts, unequal lengths
    logits = engine.step(slots, [[t] for t in next_tokens], want=[[0]] * 3)
    engine.release(slots)                           # slots and pages go back

``want[i]`` lists the places among sequence i's tokens *of this step* whose
logits are returned, in the order of the sequences and of the lists.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import Cache
from .model import Model
from .step import StepContext, StepError, StepInputs, classify

_SM_COUNT = {}


def _sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def decode_splits(batch: int, n_heads: int, max_len: int, sms: int) -> int:
    """In how many pieces a decode step cuts each sequence's keys, so that the attention
    kernel fills the GPU when batch * heads alone does not.  Depends on the longest
    context only through a power-of-two bucket, so the choice is stable while a batch grows."""
    bucket = 256
    while bucket < max_len:
        bucket *= 2
    by_len = max(1, bucket // 256)                    # at least 256 keys per piece
    by_fill = max(1, (2 * sms + batch * n_heads - 1) // (batch * n_heads))
    return int(min(by_len, by_fill, 64))


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None):
        self.model = model
        self.rt = model.rt
        needs, readers = model.cache_needs()
        self.cache = Cache(needs, readers, max_tokens, self.rt.dtype, self.rt.device, max_slots)
        self.vocab_size = model.vocab_size
        self._inputs = StepInputs(self.rt.device)
        self._heads = max([getattr(b.mixer, "n_heads", 1) for b in model.blocks] or [1])

    # -- sequences ----------------------------------------------------------------
    def start(self, n: int) -> List[int]:
        """Slots for ``n`` sequences that start together."""
        got: List[int] = []
        try:
            for _ in range(n):
                got.append(self.cache.claim())
        except Exception:
            for s in got:
                self.cache.release(s)
            raise
        return got

    def release(self, slots: Sequence[int]) -> None:
        for s in slots:
            self.cache.release(s)

    # -- the step -------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Run one step; returns float32 logits [wanted, vocab] on the device (None if nothing is wanted)."""
        slots = list(slots)
        is_prefill = classify(self.cache, slots, tokens)
        B = len(slots)
        lens = [len(t) for t in tokens]
        V = self.vocab_size
        for i, t in enumerate(tokens):
            for tok in t:
                if not (0 <= int(tok) < V):
                    raise StepError(f"sequence {i}: token id {tok} is outside the vocabulary [0, {V})")
        if want is None:
            want = [[n - 1] for n in lens]
        if len(want) != B:
            raise StepError(f"{B} sequences but {len(want)} 'want' lists")
        for i, w in enumerate(want):
            for j in w:
                if not (0 <= int(j) < lens[i]):
                    raise StepError(f"sequence {i}: wanted place {j} is outside its {lens[i]} tokens of this step")

        before = [self.cache.length(s) for s in slots]
        self.cache.grow({s: n for s, n in zip(slots, lens)})          # raises CacheFull before anything ran
        after = [b + n for b, n in zip(before, lens)]

        T = sum(lens)
        starts = np.zeros(B + 1, dtype=np.int32)
        starts[1:] = np.cumsum(lens)
        arrays: Dict[str, np.ndarray] = {
            "ids": np.fromiter((tok for t in tokens for tok in t), dtype=np.int32, count=T),
            "positions": np.concatenate([np.arange(b, b + n, dtype=np.int32) for b, n in zip(before, lens)]),
            "token_seq": np.repeat(np.arange(B, dtype=np.int32), lens),
            "seq_start": starts,
            "len_after": np.asarray(after, dtype=np.int32),
            "slot_ids": np.asarray(slots, dtype=np.int32),
            "want": np.asarray([starts[i] + j for i, w in enumerate(want) for j in w], dtype=np.int32),
        }
        max_after = max(after)
        for gi, g in enumerate(self.cache.groups):
            width = self.cache.table_width(gi, max_after)
            tab = np.zeros((B, width), dtype=np.int32)
            for i, s in enumerate(slots):
                pg = self.cache.pages(s, gi)
                tab[i, :len(pg)] = pg
            arrays[f"table{gi}"] = tab
        dev = self._inputs.upload(arrays)
        for gi, g in enumerate(self.cache.groups):
            g.table = dev[f"table{gi}"]

        ctx = StepContext(is_prefill=is_prefill, n_tokens=T, batch=B, positions=dev["positions"],
                          token_seq=dev["token_seq"], seq_start=dev["seq_start"], len_after=dev["len_after"],
                          slot_ids=dev["slot_ids"], slots=slots, seq_lens=lens, max_seq_len=max(lens),
                          max_len_after=max_after,
                          decode_splits=1 if is_prefill else decode_splits(B, self._heads, max_after,
                                                                           _sm_count(self.rt.device)))
        n_want = arrays["want"].size
        if n_want == 0:
            # nothing is asked for: the layers still run (they fill the cache), the head does not
            self.model.forward(dev["ids"], ctx, self.cache, dev["want"][:0])
            return None
        all_rows = n_want == T and bool((arrays["want"] == np.arange(T)).all())
        return self.model.forward(dev["ids"], ctx, self.cache, None if all_rows else dev["want"])

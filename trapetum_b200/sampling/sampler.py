"""From logits to the next token of every sequence of a step, on the device.

Greedy rows without a repetition penalty go through the two-stage argmax kernel;
everything else through the sampling kernel, which applies, per row and in the
reference's order (runtime/src/bin/serve.rs:327-341): repetition penalty over the
recent tokens, then argmax or a temperature/nucleus draw.  The draws come from
:func:`~trapetum_b200.sampling.params.draw_uniform`, keyed by seed, request and
token index.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import REPETITION_WINDOW, SamplingParams, draw_uniform


class Sampler:
    def __init__(self, params: SamplingParams, device):
        self.params = params
        self.device = device
        self._recent: Dict[int, Deque[int]] = {}
        self._count: Dict[int, int] = {}

    def begin(self, request: int, prompt: Sequence[int]) -> None:
        """The penalty's window starts with the end of the prompt (serve.rs:327-329)."""
        self._recent[request] = deque(list(prompt)[-REPETITION_WINDOW:], maxlen=REPETITION_WINDOW)
        self._count[request] = 0

    def end(self, request: int) -> None:
        self._recent.pop(request, None)
        self._count.pop(request, None)

    def choose(self, logits: torch.Tensor, requests: Sequence[int]) -> List[int]:
        """``logits`` float32 [rows, vocab] on the device, row i for ``requests[i]``; returns the
        chosen ids (host) and records them in the penalty windows.  If the engine already made the
        greedy choice on the device (``Engine.step(greedy=True)``), ``logits`` is that int32 tensor."""
        p = self.params
        if logits.dtype == torch.int32:
            ids = logits
        elif not p.needs_sampler:
            ids = ops.argmax(logits)
        else:
            rows = len(requests)
            f = np.empty((4, rows), dtype=np.float32)
            f[0], f[1], f[2] = p.temperature, p.top_p, p.repetition_penalty
            f[3] = [draw_uniform(p.seed, r, self._count[r]) for r in requests]
            fd = torch.from_numpy(f).to(self.device)
            recent = None
            if p.repetition_penalty > 1.0:
                rec = np.full((rows, REPETITION_WINDOW), -1, dtype=np.int32)
                for i, r in enumerate(requests):
                    w = self._recent[r]
                    rec[i, :len(w)] = list(w)
                recent = torch.from_numpy(rec).to(self.device)
            ids = ops.sample(logits, fd[0], fd[1], fd[2], fd[3], recent, nucleus=p.top_p < 1.0)
        out = ids.cpu().tolist()
        for r, t in zip(requests, out):
            self._recent[r].append(t)
            self._count[r] += 1
        return out

"""Trace replay on top of the engine: request ids to slots, steps to logits.

The program ``bin/trace_run`` is a thin shell around :class:`Replayer`, which in
turn only translates between request names and the engine's slots.  The forward
pass, the cache and the kernels are the engine's.  The reference replays a
prompt through its one-token forward and compares with stored logits in the
same spirit (runtime/src/bin/generate.rs:58-73).
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np



class Replayer:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, device: str = "cuda:0", host=None):
        import trapetum_b200 as tb
        self.engine = tb.Engine(tb.load_model(model_dir, dtype, device, host=host), max_tokens)
        self.slot_of: Dict[str, int] = {}

    def run_step(self, rec: dict) -> Optional[np.ndarray]:
        entries = rec.get("entries", [])
        logits = None
        if entries:
            ids = [str(e["id"]) for e in entries]
            new = [i for i in ids if i not in self.slot_of]
            if new and len(new) != len(ids):
                raise ValueError(f"step {rec.get('step')}: requests {new} start while others of the step go on")
            if new:
                for i, s in zip(ids, self.engine.start(len(ids))):
                    self.slot_of[i] = s
            out = self.engine.step([self.slot_of[i] for i in ids], [e["tokens"] for e in entries],
                                   [e.get("want", []) for e in entries])
            if out is not None:
                logits = out.float().cpu().numpy()
            self.engine.check_kernels()          # logits of a kernel that gave up waiting must not be written
        for i in rec.get("end", []):
            i = str(i)
            if i not in self.slot_of:
                raise ValueError(f"step {rec.get('step')}: request '{i}' ends but was never started")
            self.engine.release([self.slot_of.pop(i)])
        return logits

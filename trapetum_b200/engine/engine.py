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
from ..csrc import ops
from .model import Model
from .step import StepContext, StepError, StepInputs, classify

_SM_COUNT = {}


def _sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def unevenness(lens: Sequence[int]) -> int:
    """How much a batch's context lengths differ, in quarters: 0 if their sum is at least three quarters of
    batch x longest, 1 from a half on, 2 from a quarter on, else 3.  Work dealt out by the longest sequence
    leaves that share of the GPU idle; decode attention weighs it against what dealing the pages out as one
    stream costs (``ops.attn_decode``).  Launch shapes depend on the lengths only through this and the bucket."""
    if len(lens) <= 1:
        return 0
    full = len(lens) * max(lens)
    return max(0, min(3, 3 - (4 * sum(lens)) // full)) if full > 0 else 0


def uneven_lengths(lens: Sequence[int]) -> bool:
    """Whether the lengths differ at all in the sense of :func:`unevenness`."""
    return unevenness(lens) > 0


def len_bucket(max_len: int) -> int:
    """The smallest power of two (at least 256) that is not below ``max_len``.  Launch shapes of a decode
    step (how attention cuts the keys) depend on the longest context only through this bucket, so they stay
    the same for many steps and a captured graph stays valid."""
    b = 256
    while b < max_len:
        b *= 2
    return b


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None, use_graphs: bool = True):
        self.model = model
        self.rt = model.rt
        needs, readers = model.cache_needs()
        self.cache = Cache(needs, readers, max_tokens, self.rt.dtype, self.rt.device, max_slots)
        self.vocab_size = model.vocab_size
        self._inputs = StepInputs(self.rt.device)
        # CUDA graphs for decode steps: only if every part says that its launches depend on nothing
        # that lives on the host (a part that reads ctx.slots in Python, for one, does not qualify)
        self.use_graphs = use_graphs and self.rt.device.type == "cuda"
        self._graph_safe = all(getattr(p, "graph_safe", False) for b in model.blocks for p in (b, b.mixer, b.feed_forward))
        self._decode: Dict[tuple, "_DecodeShape"] = {}
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs and self._graph_safe else None

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
             want: Optional[Sequence[Sequence[int]]] = None, borrow: bool = False,
             greedy: bool = False) -> Optional[torch.Tensor]:
        """Run one step; returns float32 logits [wanted, vocab] on the device (None if nothing is wanted).

        ``borrow=True`` lets the result alias a buffer that the next step overwrites (the generation
        loop consumes the logits at once and saves the copy).  ``greedy=True`` returns, instead of the
        logits, the int32 ids of the largest logit at each wanted place (the smallest id on a tie),
        chosen on the device; in a decode step the choice is part of the captured graph."""
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
        after = [b + n for b, n in zip(before, lens)]
        cap = self.model.spec.max_positions
        for i, n in enumerate(after):
            if n > cap:
                raise StepError(f"sequence {i}: {n} tokens after this step, the model has {cap} positions")
        growth = {s: n for s, n in zip(slots, lens)}
        self.cache.grow(growth)                                       # raises CacheFull before anything ran
        try:
            return self._run(slots, tokens, want, is_prefill, lens, before, after, borrow, greedy)
        except BaseException:
            # the step did not run to its end: the cache must not claim tokens whose keys were never written
            self.cache.shrink(growth)
            raise

    def step_tokens(self, slots: Sequence[int], tokens: Sequence[Sequence[int]]) -> List[int]:
        """One step of a generation loop: host token lists in, each sequence's greedy next token out (host ints)."""
        return self.step(slots, tokens, borrow=True, greedy=True).cpu().tolist()

    @property
    def graphs_captured(self) -> int:
        """How many decode-step shapes run as captured graphs by now."""
        return sum(1 for d in self._decode.values() if d.graph is not None)

    @property
    def last_h2d_bytes(self) -> int:
        """Bytes of the last decode step's one host-to-device copy (its integer inputs and page tables)."""
        return max((d.h2d_bytes for d in self._decode.values()), default=0)

    def check_kernels(self) -> None:
        """Raise :class:`~trapetum_b200.csrc.ops.KernelError` if a kernel's bounded wait has run out since
        the last check (its results are then garbage).  Synchronises the device, so callers place it where they
        wait for the device anyway: the generation loop at the end of a batch, trace replay after a step."""
        err = ops.kernel_errors()
        if err:
            raise ops.KernelError(f"a kernel gave up waiting and its results are not valid: {err}")

    def _run(self, slots, tokens, want, is_prefill, lens, before, after, borrow, greedy):
        B = len(slots)
        if not is_prefill and self.use_graphs and self._graph_safe:
            return self._decode_step(slots, tokens, want, before, after, borrow, greedy)

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
            arrays[f"table{gi}"] = self._table(gi, slots, self.cache.table_width(gi, max_after))
        dev = self._inputs.upload(arrays)
        for gi, g in enumerate(self.cache.groups):
            g.table = dev[f"table{gi}"]

        ctx = StepContext(is_prefill=is_prefill, n_tokens=T, batch=B, positions=dev["positions"],
                          token_seq=dev["token_seq"], seq_start=dev["seq_start"], len_after=dev["len_after"],
                          slot_ids=dev["slot_ids"], slots=slots, seq_lens=lens, max_seq_len=max(lens),
                          max_len_after=max_after, len_bucket=len_bucket(max_after),
                          uneven=0 if is_prefill else unevenness(after))
        n_want = arrays["want"].size
        if n_want == 0:
            # nothing is asked for: the layers still run (they fill the cache), the head does not
            self.model.forward(dev["ids"], ctx, self.cache, dev["want"][:0])
            return None
        all_rows = n_want == T and bool((arrays["want"] == np.arange(T)).all())
        logits = self.model.forward(dev["ids"], ctx, self.cache, None if all_rows else dev["want"])
        return ops.argmax(logits) if greedy else logits

    def _table(self, gi: int, slots: Sequence[int], width: int) -> np.ndarray:
        tab = np.zeros((len(slots), width), dtype=np.int32)
        for i, s in enumerate(slots):
            pg = self.cache.pages(s, gi)
            tab[i, :len(pg)] = pg
        return tab

    # -- one token per sequence, as a CUDA graph ---------------------------------------
    def _decode_step(self, slots, tokens, want, before, after, borrow, greedy=False):
        """A decode step's launches do not depend on the tokens, the positions or the pages, only on
        the batch size and on the bucket of the longest context: the inputs live in buffers of a fixed layout,
        the first step of a shape runs eagerly (it also sets up every kernel), the second is captured
        into a CUDA graph, and from then on a step is one copy of the inputs and one graph launch."""
        B = len(slots)
        max_after = max(after)
        bucket = len_bucket(max_after)
        uneven = unevenness(after)
        key = (B, bucket, uneven)
        dg = self._decode.get(key)
        if dg is None:
            dg = self._decode[key] = _DecodeShape(B, bucket, self, uneven)
        dg.fill(self, slots, [t[0] for t in tokens], before, after)
        for gi, g in enumerate(self.cache.groups):
            g.table = dg.dev[f"table{gi}"]
        dg.hits += 1
        if dg.graph is None and dg.hits >= 2:
            ctx = dg.context(slots, max_after)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                dg.logits = self.model.forward(dg.dev["ids"], ctx, self.cache, None)
                dg.greedy = ops.argmax(dg.logits)      # the greedy choice rides along in the graph
            dg.graph = graph
        if dg.graph is not None:
            dg.graph.replay()
            logits, ids = dg.logits, dg.greedy
            ops.count_launches(dg.n_kernels)
        else:
            n0 = ops.launches()
            logits = self.model.forward(dg.dev["ids"], dg.context(slots, max_after), self.cache, None)
            ids = ops.argmax(logits)
            dg.n_kernels = ops.launches() - n0
        rows = [i for i, w in enumerate(want) for _ in w]
        if not rows:
            return None
        if rows == list(range(B)):
            out = ids if greedy else logits
            return out if (borrow or dg.graph is None) else out.clone()
        idx = torch.tensor(rows, dtype=torch.int32, device=self.rt.device)
        return ops.argmax(ops.gather_rows(logits, idx)) if greedy else ops.gather_rows(logits, idx)


class _DecodeShape:
    """The fixed-layout inputs, and later the graph, of decode steps of one batch size and length bucket."""

    def __init__(self, B: int, bucket: int, engine: "Engine", uneven: int = 0):
        self.B, self.bucket, self.uneven = B, bucket, uneven
        self.graph = None
        self.logits = None
        self.greedy = None
        self.hits = 0
        self._tables_of = None                # (slots, cache epoch) the device tables were last written for
        self.n_kernels = 0
        cache = engine.cache
        cap = min(engine.model.spec.max_positions, cache.max_tokens)
        self.widths = [cache.table_width(gi, cap) for gi in range(len(cache.groups))]
        names = [("ids", (B,)), ("positions", (B,)), ("token_seq", (B,)), ("seq_start", (B + 1,)),
                 ("len_after", (B,)), ("slot_ids", (B,))] + [(f"table{gi}", (B, w)) for gi, w in enumerate(self.widths)]
        off, self.layout = 0, {}
        for name, shape in names:
            n = int(np.prod(shape))
            self.layout[name] = (off, shape)
            off += (n + 3) & ~3
        dev = engine.rt.device
        self.host = torch.zeros(off, dtype=torch.int32).pin_memory()
        self.buf = torch.zeros(off, dtype=torch.int32, device=dev)
        self.hv = {name: self.host.numpy()[o:o + int(np.prod(shape))].reshape(shape) for name, (o, shape) in self.layout.items()}
        self.dev = {name: self.buf[o:o + int(np.prod(shape))].view(shape) for name, (o, shape) in self.layout.items()}
        self.hv["token_seq"][:] = np.arange(B)
        self.hv["seq_start"][:] = np.arange(B + 1)
        self.copied = None
        self.h2d_bytes = off * 4

    def fill(self, engine, slots, toks, before, after) -> None:
        if self.copied is not None:
            self.copied.synchronize()              # the last copy has left the host buffer
        hv = self.hv
        hv["ids"][:] = toks
        hv["positions"][:] = before
        hv["len_after"][:] = after
        hv["slot_ids"][:] = slots
        # The page tables change only when the batch's slots change or when any slot or page of the cache
        # changes hands (the cache counts those events): two batches may hold the same slots with the same
        # numbers of pages and yet other pages.
        cache = engine.cache
        key = (tuple(slots), cache.epoch)
        if key != self._tables_of:
            self._tables_of = key
            for gi, w in enumerate(self.widths):
                t = hv[f"table{gi}"]
                for i, s in enumerate(slots):
                    pg = cache.pages(s, gi)
                    t[i, :len(pg)] = pg
        self.buf.copy_(self.host, non_blocking=True)
        self.copied = torch.cuda.Event()
        self.copied.record()

    def context(self, slots, max_after) -> StepContext:
        d = self.dev
        return StepContext(is_prefill=False, n_tokens=self.B, batch=self.B, positions=d["positions"],
                           token_seq=d["token_seq"], seq_start=d["seq_start"], len_after=d["len_after"],
                           slot_ids=d["slot_ids"], slots=list(slots), seq_lens=[1] * self.B, max_seq_len=1,
                           max_len_after=max_after, len_bucket=self.bucket, uneven=self.uneven)

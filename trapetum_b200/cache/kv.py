"""The cache: keys and values per layer call, pages per sequence, state per slot.

Every schedule entry that owns a cache declares what it needs
(:class:`~trapetum_b200.parts.base.KVNeed` or ``StateNeed``).  Entries with the
same key/value geometry and the same window form a *group*; a group has one
allocation ``[lines, pages, kv_heads, PAGE_ROWS, head_dim]`` for keys, one for
values, and one page pool, because all its lines grow in step: page ``p`` of a
sequence is page ``p`` in every line of the group.

* A group without a window keeps every token: row = position.
* A group with window W is a ring of ``ring_rows = ceil(W / PAGE_ROWS) * PAGE_ROWS``
  rows per sequence: row = position mod ring_rows.  It never holds more than
  ``ring_rows`` tokens of a sequence, whatever the sequence's length.

A sequence takes a slot when it starts and pages as it grows; :meth:`release`
gives all of it back, and the next sequence reuses the numbers.  Stale keys in a
reused page are never read: every reader is bounded by the sequence's own length.

``StateNeed`` entries get ``[max_slots, *shape]`` of their dtype each, addressed by slot
and zeroed when the slot is taken.  Gemma-2 has none; the area exists so that a
mixer with a recurrent state has a place to keep it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..csrc.ops import PAGE_ROWS
from ..parts.base import KVNeed, StateNeed
from .slots import CacheError, CacheFull, Pool


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_ROWS - 1) // PAGE_ROWS


@dataclass
class KVGroup:
    need: KVNeed
    entries: List[int]                       # schedule entries (cache owners) in this group
    ring_rows: int                           # 0: keeps everything
    pool: Pool
    k: torch.Tensor                          # [lines, pages, kv_heads, PAGE_ROWS, head_dim]
    v: torch.Tensor
    table: Optional[torch.Tensor] = None     # device int32 [batch rows, width], owned by the engine's batch

    def rows_held(self, length: int) -> int:
        return min(length, self.ring_rows) if self.ring_rows else length


@dataclass
class KVLineView:
    """What a mixer call sees of the cache."""
    k: torch.Tensor                          # [pages, kv_heads, PAGE_ROWS, head_dim]
    v: torch.Tensor
    page_table: Optional[torch.Tensor]       # int32 [batch, width] of the running batch
    ring_rows: int
    window: Optional[int]
    entry: int                               # the owning schedule entry
    owner: bool                              # this call writes the line
    shared: bool                             # some later call reads this line


@dataclass
class StateView:
    """Per-slot state of one schedule entry: ``data[slot]`` is the sequence's state."""
    data: torch.Tensor                       # [max_slots, *shape] of the need's dtype
    entry: int


class Cache:
    def __init__(self, needs: Dict[int, object], readers: Dict[int, List[int]], max_tokens: int,
                 dtype: torch.dtype, device, max_slots: Optional[int] = None):
        """``needs``: owning schedule entry -> KVNeed | StateNeed.  ``readers``: owning
        entry -> entries that read its cache.  ``max_tokens``: the most tokens that live
        sequences hold at any time, each sequence's count rounded up to PAGE_ROWS."""
        if max_tokens <= 0:
            raise ValueError(f"cache: max_tokens must be positive, got {max_tokens}")
        self.dtype, self.device = dtype, torch.device(device)
        self.n_pages = pages_for(max_tokens)
        self.max_tokens = self.n_pages * PAGE_ROWS
        self.max_slots = min(self.n_pages, max_slots or 1024)
        self.slots = Pool(self.max_slots, "slot")
        self.groups: List[KVGroup] = []
        self.entry_group: Dict[int, Tuple[int, int]] = {}     # entry -> (group index, line index)
        self.states: Dict[int, torch.Tensor] = {}
        self.readers = readers
        by_key: Dict[Tuple, List[int]] = {}
        for e in sorted(needs):
            need = needs[e]
            if isinstance(need, KVNeed):
                by_key.setdefault((need.n_kv_heads, need.head_dim, need.window), []).append(e)
            elif isinstance(need, StateNeed):
                self.states[e] = torch.zeros((self.max_slots,) + tuple(need.shape), dtype=need.dtype,
                                             device=self.device)
            elif need is not None:
                raise TypeError(f"schedule entry {e}: a cache need must be KVNeed, StateNeed or None, got {need!r}")
        for (nkv, hd, window), entries in by_key.items():
            ring = pages_for(window) * PAGE_ROWS if window else 0
            shape = (len(entries), self.n_pages, nkv, PAGE_ROWS, hd)
            # a ring never holds more than ring_rows per sequence, so its pool can be smaller
            n_pages = min(self.n_pages, self.max_slots * (ring // PAGE_ROWS)) if ring else self.n_pages
            shape = (len(entries), n_pages, nkv, PAGE_ROWS, hd)
            g = KVGroup(KVNeed(nkv, hd, window), entries, ring, Pool(n_pages, "page"),
                        torch.empty(shape, dtype=dtype, device=self.device),
                        torch.empty(shape, dtype=dtype, device=self.device))
            for i, e in enumerate(entries):
                self.entry_group[e] = (len(self.groups), i)
            self.groups.append(g)
        self._len: Dict[int, int] = {}                         # slot -> tokens held
        self._pages: Dict[int, List[List[int]]] = {}           # slot -> per group page list
        # Counts every change of who holds which slot or page.  A page table written for (slots, epoch) stays
        # right exactly as long as neither changes: equal page COUNTS do not mean equal page NUMBERS once
        # sequences have ended and others have started.
        self.epoch = 0

    # -- sequences -------------------------------------------------------------
    def claim(self) -> int:
        """Take a slot for a new sequence (length 0, state zeroed)."""
        (slot,) = self.slots.take(1)
        self.epoch += 1
        self._len[slot] = 0
        self._pages[slot] = [[] for _ in self.groups]
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def length(self, slot: int) -> int:
        self._held(slot)
        return self._len[slot]

    def pages(self, slot: int, group: int) -> List[int]:
        self._held(slot)
        return self._pages[slot][group]

    def grow(self, growth: Dict[int, int]) -> None:
        """Make room for ``growth[slot]`` more tokens per slot: all of it or nothing."""
        want: List[Tuple[int, int, int]] = []                  # (slot, group, pages to add)
        per_group = [0] * len(self.groups)
        for slot, n in growth.items():
            self._held(slot)
            if n < 0:
                raise CacheError(f"slot {slot}: cannot grow by {n}")
            new_len = self._len[slot] + n
            for gi, g in enumerate(self.groups):
                add = pages_for(g.rows_held(new_len)) - len(self._pages[slot][gi])
                if add > 0:
                    want.append((slot, gi, add))
                    per_group[gi] += add
        for gi, g in enumerate(self.groups):
            if per_group[gi] > g.pool.free:
                held = sum(self._len.values())
                raise CacheFull(f"the cache is full: this step needs {per_group[gi]} more pages of {PAGE_ROWS} tokens, "
                                f"{g.pool.free} of {g.pool.capacity} are free ({len(self._len)} live sequences hold "
                                f"{held} tokens; the cache was sized for {self.max_tokens})")
        for slot, gi, add in want:
            self._pages[slot][gi].extend(self.groups[gi].pool.take(add))
        if want:
            self.epoch += 1
        for slot, n in growth.items():
            self._len[slot] += n

    def shrink(self, growth: Dict[int, int]) -> None:
        """Undo a :meth:`grow` whose step did not run: the lengths go back and the pages that only the
        growth needed are returned.  Rows of the undone tokens may have been written; no reader reaches them
        (every reader is bounded by the length), and in a ring the rows they replaced lay outside every later
        query's window."""
        for slot, n in growth.items():
            self._held(slot)
            if n < 0 or n > self._len[slot]:
                raise CacheError(f"slot {slot}: cannot shrink {self._len[slot]} tokens by {n}")
        for slot, n in growth.items():
            self._len[slot] -= n
            for gi, g in enumerate(self.groups):
                keep = pages_for(g.rows_held(self._len[slot]))
                extra = self._pages[slot][gi][keep:]
                if extra:
                    del self._pages[slot][gi][keep:]
                    g.pool.give_back(extra)
        self.epoch += 1

    def release(self, slot: int) -> None:
        self._held(slot)
        for gi, g in enumerate(self.groups):
            g.pool.give_back(self._pages[slot][gi])
        del self._pages[slot], self._len[slot]
        self.slots.give_back([slot])
        self.epoch += 1

    def live_slots(self) -> List[int]:
        return sorted(self._len)

    def _held(self, slot: int) -> None:
        if slot not in self._len:
            raise CacheError(f"slot {slot} is not held by any sequence")

    def check(self) -> None:
        """Bookkeeping invariants: no page lost, none held twice."""
        self.slots.check()
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen = []
            for slot in self._len:
                seen.extend(self._pages[slot][gi])
            if len(set(seen)) != len(seen):
                raise CacheError(f"group {gi}: a page belongs to two sequences")
            if len(seen) != g.pool.held:
                raise CacheError(f"group {gi}: {g.pool.held} pages are taken, sequences hold {len(seen)}")

    # -- views ------------------------------------------------------------------
    def table_width(self, group: int, max_len: int) -> int:
        return max(1, pages_for(self.groups[group].rows_held(max_len)))

    def line(self, entry: int, owner_entry: int) -> KVLineView:
        gi, li = self.entry_group[owner_entry]
        g = self.groups[gi]
        return KVLineView(g.k[li], g.v[li], g.table, g.ring_rows, g.need.window, owner_entry,
                          owner=(entry == owner_entry), shared=bool(self.readers.get(owner_entry)))

    def view(self, entry: int, owner_entry: int):
        if owner_entry in self.entry_group:
            return self.line(entry, owner_entry)
        if owner_entry in self.states:
            return StateView(self.states[owner_entry], owner_entry)
        return None

    def bytes_per_token(self) -> int:
        """Key and value bytes one token adds across all groups (rings add nothing past their size)."""
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.need.n_kv_heads * g.need.head_dim * es for g in self.groups)

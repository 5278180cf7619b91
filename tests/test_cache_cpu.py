"""The cache's bookkeeping (no GPU): no slot or page is lost, held twice or freed twice."""
import random

import pytest
import torch

from trapetum_b200.cache import Cache, CacheError, CacheFull, Pool, pages_for
from trapetum_b200.csrc.ops import PAGE_ROWS
from trapetum_b200.parts import KVNeed, StateNeed


def make(max_tokens=PAGE_ROWS * 16, window=None, max_slots=None, state=False):
    needs = {0: KVNeed(2, 16, window), 1: KVNeed(2, 16, None), 2: KVNeed(2, 16, window), 3: KVNeed(2, 16, None)}
    if state:
        needs[4] = StateNeed((3, 5))
    return Cache(needs, {1: [5]}, max_tokens, torch.float32, "cpu", max_slots)


def test_pool_basics():
    p = Pool(4, "page")
    a = p.take(3)
    assert a == [0, 1, 2] and p.free == 1 and p.held == 3
    with pytest.raises(CacheFull):
        p.take(2)
    p.give_back([1])
    assert p.take(1) == [1]                      # the lowest free number is used again
    with pytest.raises(CacheError, match="not held"):
        p.give_back([3])
    p.give_back([0])
    with pytest.raises(CacheError, match="not held"):
        p.give_back([0])                         # freed twice
    with pytest.raises(CacheError, match="twice"):
        p.give_back([1, 1])
    p.check()


def test_groups_by_need():
    c = make(window=100)
    assert len(c.groups) == 2
    ring = [g for g in c.groups if g.ring_rows][0]
    full = [g for g in c.groups if not g.ring_rows][0]
    assert ring.entries == [0, 2] and full.entries == [1, 3]
    assert ring.ring_rows == 2 * PAGE_ROWS                       # 100 rounded up to whole pages
    assert full.k.shape == (2, 16, 2, PAGE_ROWS, 16)
    assert c.line(5, 1).owner is False and c.line(1, 1).owner and c.line(1, 1).shared and not c.line(3, 3).shared


def test_grow_release_reuse():
    c = make(window=100)
    s0, s1 = c.claim(), c.claim()
    c.grow({s0: 70, s1: 5})
    full = next(i for i, g in enumerate(c.groups) if not g.ring_rows)
    ring = 1 - full
    assert len(c.pages(s0, full)) == 2 and len(c.pages(s1, full)) == 1 and c.length(s0) == 70
    c.grow({s0: 200})
    assert len(c.pages(s0, full)) == pages_for(270) and len(c.pages(s0, ring)) == 2   # the ring stops growing
    c.check()
    held = set(c.pages(s0, full))
    c.release(s0)
    with pytest.raises(CacheError, match="not held"):
        c.release(s0)
    with pytest.raises(CacheError):
        c.length(s0)
    s2 = c.claim()
    assert s2 == s0                                                # the slot number is used again
    c.grow({s2: 64 * 3})
    assert set(c.pages(s2, full)) & held                           # and so are its pages
    c.check()
    c.release(s1); c.release(s2); c.check()
    assert all(g.pool.held == 0 for g in c.groups) and c.slots.held == 0


def test_full_cache_refuses_whole_step():
    c = make(max_tokens=PAGE_ROWS * 4)
    a, b = c.claim(), c.claim()
    c.grow({a: PAGE_ROWS * 2, b: PAGE_ROWS})
    with pytest.raises(CacheFull, match="full"):
        c.grow({a: 1, b: PAGE_ROWS})                               # needs 2 pages, 1 is free
    assert c.length(a) == PAGE_ROWS * 2 and c.length(b) == PAGE_ROWS    # nothing was taken
    c.check()
    c.grow({a: 1})
    c.check()


def test_max_tokens_counts_whole_pages_per_sequence():
    c = make(max_tokens=PAGE_ROWS * 3)
    s = [c.claim() for _ in range(3)]
    c.grow({x: 1 for x in s})                                     # 3 tokens hold 3 pages
    with pytest.raises(CacheFull):
        c.claim() if c.slots.free == 0 else c.grow({s[0]: PAGE_ROWS})
    c.check()


def test_state_area_is_zeroed_at_claim():
    c = make(state=True, max_slots=4)
    st = c.view(4, 4)
    assert st.data.shape == (4, 3, 5) and st.data.dtype == torch.float32
    s = c.claim()
    st.data[s] += 7
    c.release(s)
    assert c.claim() == s and float(st.data[s].abs().sum()) == 0.0


def test_random_churn_keeps_invariants():
    rnd = random.Random(0)
    c = make(max_tokens=PAGE_ROWS * 40, window=130)
    live = {}
    for step in range(600):
        r = rnd.random()
        if r < 0.25 and c.slots.free:
            live[c.claim()] = 0
        elif r < 0.8 and live:
            s = rnd.choice(list(live))
            n = rnd.choice([1, 1, 1, 7, 64, 200])
            try:
                c.grow({s: n})
                live[s] += n
            except CacheFull:
                pass
        elif live:
            s = rnd.choice(list(live))
            c.release(s)
            del live[s]
        c.check()
        assert c.live_slots() == sorted(live)
        for s, n in live.items():
            assert c.length(s) == n
            for gi, g in enumerate(c.groups):
                assert len(c.pages(s, gi)) == pages_for(g.rows_held(n))
    for s in list(live):
        c.release(s)
    c.check()
    assert all(g.pool.free == g.pool.capacity for g in c.groups)


def test_epoch_counts_every_change_of_hands():
    """Two batches can hold the same slots with the same numbers of pages and yet other pages: whoever keeps
    a page table must be able to tell (the epoch differs)."""
    c = make(max_tokens=PAGE_ROWS * 8)
    a = [c.claim(), c.claim()]
    c.grow({a[0]: 40, a[1]: 40})
    for _ in range(30):
        c.grow({a[0]: 1, a[1]: 1})
    tables_a = [[list(c.pages(s, g)) for g in range(len(c.groups))] for s in a]
    seen = c.epoch
    for s in a:
        c.release(s)
    b = [c.claim(), c.claim()]
    c.grow({b[0]: 70, b[1]: 70})
    tables_b = [[list(c.pages(s, g)) for g in range(len(c.groups))] for s in b]
    assert b == a and [[len(p) for p in t] for t in tables_b] == [[len(p) for p in t] for t in tables_a]
    assert tables_b != tables_a                # same slots, same counts, other pages
    assert c.epoch != seen
    e = c.epoch
    c.grow({b[0]: 1, b[1]: 1})                 # no new page: nothing changed hands
    assert c.epoch == e
    c.grow({b[0]: 64, b[1]: 64})
    assert c.epoch != e


def test_shrink_undoes_a_grow():
    c = make(max_tokens=PAGE_ROWS * 8, window=100)
    s = c.claim()
    c.grow({s: 70})
    before = [list(c.pages(s, g)) for g in range(len(c.groups))]
    free = [g.pool.free for g in c.groups]
    c.grow({s: 130})
    c.shrink({s: 130})
    assert c.length(s) == 70 and [list(c.pages(s, g)) for g in range(len(c.groups))] == before
    assert [g.pool.free for g in c.groups] == free
    c.check()
    with pytest.raises(CacheError):
        c.shrink({s: 71})
    c.shrink({s: 70})
    assert c.length(s) == 0 and all(g.pool.held == 0 for g in c.groups)
    c.release(s)
    c.check()

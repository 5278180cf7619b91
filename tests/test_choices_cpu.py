"""Host-side choices that shape launches (no GPU): the length bucket and the number of key splits."""
from trapetum_b200.csrc.ops import choose_decode_splits
from trapetum_b200.engine import len_bucket


def test_len_bucket_is_a_power_of_two_not_below():
    assert len_bucket(1) == 256 and len_bucket(256) == 256 and len_bucket(257) == 512
    assert len_bucket(8192) == 8192 and len_bucket(8193) == 16384
    for n in (3, 100, 1000, 5000):
        b = len_bucket(n)
        assert b >= n and b & (b - 1) == 0


def test_decode_splits():
    # one sequence: many pieces, to put a CTA on as many SMs as the pages allow (at least 4 pages each)
    assert choose_decode_splits(1, 4, 128, 148) == 31
    # a short context is not cut
    assert choose_decode_splits(8, 4, 4, 148) == 1 and choose_decode_splits(1, 4, 7, 148) == 1
    # 32 (sequence, kv head) pairs on 148 SMs: four pieces fill one round
    assert choose_decode_splits(8, 4, 128, 148) == 4
    # 256 pairs: one piece would leave most of a second round idle
    assert choose_decode_splits(64, 4, 128, 148) == 4
    for batch in (1, 3, 8, 64, 200):
        for pages in (1, 9, 64, 128, 1000):
            s = choose_decode_splits(batch, 4, pages, 148)
            assert 1 <= s <= 64 and (s == 1 or pages // s >= 4)


def test_uneven_lengths():
    """The engine tells the kernels when a batch's contexts differ so much that cutting every sequence alike
    would leave most CTAs with nothing to do; it is part of the key of a captured decode step."""
    from trapetum_b200.engine.engine import uneven_lengths
    assert not uneven_lengths([8000])                       # one sequence is never uneven
    assert not uneven_lengths([8000, 8000, 7000, 8192])
    assert uneven_lengths([8000, 100, 100, 100])
    assert uneven_lengths([1, 1, 1, 64])
    assert not uneven_lengths([3, 3, 4])

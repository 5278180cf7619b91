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


def test_unevenness_and_the_partition_it_chooses():
    """The engine tells the kernels how much a batch's contexts differ (in quarters of batch x longest that are
    empty); it is part of the key of a captured decode step.  Decode attention deals its pages out as one stream
    only where that saves more than a streaming launch costs."""
    from trapetum_b200.csrc.ops import decode_partition_is_stream
    from trapetum_b200.engine.engine import uneven_lengths, unevenness
    assert unevenness([8000]) == 0                          # one sequence is never uneven
    assert unevenness([8000, 8000, 7000, 8192]) == 0
    assert unevenness([3, 3, 4]) == 0
    assert unevenness([4, 4, 4, 4]) == 0 and unevenness([4, 4, 4, 0]) == 0 and unevenness([4, 4, 3, 0]) == 1
    assert unevenness([8, 8, 0, 0]) == 1 and unevenness([8, 7, 0, 0]) == 2 and unevenness([8, 0, 0, 0]) == 2
    assert unevenness([8, 0, 0, 0, 0]) == 3
    assert unevenness([8000, 100, 100, 100]) == 2 and unevenness([8000] + [64] * 7) == 3
    assert unevenness([1, 1, 1, 64]) == 2
    assert uneven_lengths([8000, 100, 100, 100]) and not uneven_lengths([5, 5])
    # prompts of 64 to 2,048 tokens in a batch of 8 (sum 8,305 of 8 x 1,919), 9B heads: pieces of 16 pages, a
    # quarter of which a stream would save: the sequences are cut
    lens = [1555, 532, 1206, 836, 1919, 144, 1149, 964]
    assert unevenness(lens) == 1
    assert not decode_partition_is_stream(8, 8, 32, choose_decode_splits(8, 8, 32, 148), 1, 148)
    # one long sequence among short ones: 32-page pieces, three quarters saved: one stream
    assert decode_partition_is_stream(8, 4, 128, choose_decode_splits(8, 4, 128, 148), 3, 148)
    # equal lengths: a stream only where the pieces would take more than two rounds of CTAs
    assert not decode_partition_is_stream(8, 4, 128, 4, 0, 148) and not decode_partition_is_stream(64, 4, 32, 1, 0, 148)
    assert decode_partition_is_stream(64, 16, 32, 1, 0, 148)

"""The generation loop's decisions (no GPU): batching, stopping, the draws, and the loop itself
driven against a stand-in engine."""
import pytest
import torch

from trapetum_b200.cache import Cache
from trapetum_b200.csrc.ops import PAGE_ROWS
from trapetum_b200.engine import generate as gen
from trapetum_b200.engine.generate import plan_batches, should_stop
from trapetum_b200.parts import KVNeed
from trapetum_b200.sampling import SamplingParams, draw_uniform


def test_plan_batches_by_count_and_by_room():
    assert plan_batches([5, 11, 17, 64, 200], 8, 2, 64 * 100, 8192) == [[0, 1], [2, 3], [4]]
    # 3 pages each (130 + 8 tokens): a cache of 7 pages takes two at a time
    assert plan_batches([130] * 5, 8, 64, 7 * PAGE_ROWS, 8192) == [[0, 1], [2, 3], [4]]
    with pytest.raises(ValueError, match="request 1"):
        plan_batches([5, 300], 8, 4, 2 * PAGE_ROWS, 8192)
    with pytest.raises(ValueError, match="empty"):
        plan_batches([0], 8, 4, 1024, 8192)
    with pytest.raises(ValueError, match="positions"):
        plan_batches([9000], 8, 4, 1 << 20, 8192)


def test_should_stop():
    assert should_stop(7, 0, 10, {7}, 5, 100) == "stop"
    assert should_stop(3, 4, 10, {7}, 5, 100) == "length"
    assert should_stop(3, 3, 10, {7}, 5, 100) is None
    assert should_stop(3, 0, 98, {7}, 5, 100) is None
    assert should_stop(3, 0, 99, {7}, 5, 100) == "context"


def test_draws_are_reproducible_and_in_range():
    a = [draw_uniform(3, r, i) for r in range(4) for i in range(50)]
    b = [draw_uniform(3, r, i) for r in range(4) for i in range(50)]
    assert a == b and all(0.0 <= u < 1.0 for u in a)
    assert len(set(a)) > 190
    assert 0.4 < sum(a) / len(a) < 0.6
    assert draw_uniform(3, 0, 0) != draw_uniform(4, 0, 0)
    assert all(float(torch.tensor(u, dtype=torch.float32)) == u for u in a)     # exact in float32


def test_sampling_params():
    assert SamplingParams().greedy and not SamplingParams().needs_sampler
    assert SamplingParams(repetition_penalty=1.3).needs_sampler
    assert not SamplingParams(temperature=0.7).greedy
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)


class _Spec:
    max_positions = 40
    stop_ids = (3,)


class _Model:
    spec = _Spec()


class _Rt:
    device = "cpu"


class FakeEngine:
    """Stands in for the engine: the next token of a sequence is (sum of its tokens) mod 11.
    Records every step and checks what the loop may assume."""

    def __init__(self, max_tokens=PAGE_ROWS * 8):
        self.cache = Cache({0: KVNeed(1, 8, None)}, {}, max_tokens, torch.float32, "cpu")
        self.model, self.rt = _Model(), _Rt()
        self.sums, self.steps = {}, []
        self.checks = []                       # live sequences at each look at the kernels' error words

    def check_kernels(self):
        self.checks.append(len(self.cache.live_slots()))

    def start(self, n):
        return [self.cache.claim() for _ in range(n)]

    def release(self, slots):
        for s in slots:
            self.cache.release(s)
            del self.sums[s]

    def step(self, slots, tokens, want=None, borrow=False, greedy=False):
        first = all(self.cache.length(s) == 0 for s in slots)
        assert first or all(len(t) == 1 and self.cache.length(s) > 0 for s, t in zip(slots, tokens))
        self.cache.grow({s: len(t) for s, t in zip(slots, tokens)})
        self.steps.append((list(slots), [len(t) for t in tokens], first))
        logits = torch.zeros(len(slots), 11)
        for i, (s, t) in enumerate(zip(slots, tokens)):
            self.sums[s] = self.sums.get(s, 0) + sum(t)
            logits[i, self.sums[s] % 11] = 1.0
        return logits.argmax(-1).to(torch.int32) if greedy else logits


class FakeSampler:
    def __init__(self, params, device):
        pass

    def begin(self, r, p): pass
    def end(self, r): pass

    def choose(self, logits, requests):
        return logits.tolist() if logits.dtype == torch.int32 else logits.argmax(-1).tolist()


def expected(prompt, n, stops=(3,)):
    out, s = [], sum(prompt)
    for _ in range(n):
        t = s % 11
        if t in stops:
            break
        out.append(t); s += t
    return out


def test_loop_against_a_stand_in(monkeypatch):
    monkeypatch.setattr(gen, "Sampler", FakeSampler)
    eng = FakeEngine()
    prompts = [[1, 2], [5], [4, 4, 4], [2, 2, 2, 2, 1], [10]]
    outs = gen.generate(eng, prompts, max_tokens=6, max_batch=2)
    assert outs == [expected(p, 6) for p in prompts]
    assert any(len(o) < 6 for o in outs) and any(len(o) == 6 for o in outs)     # some stop early, some do not
    # batches of two, one after another; every slot went back
    assert eng.steps[0][1] == [2, 1] and eng.cache.live_slots() == []
    eng.cache.check()
    assert [s[1] for s in eng.steps if s[2]] == [[2, 1], [3, 5], [1]]
    # within a batch the set of stepped slots only shrinks: a finished sequence never comes back
    for prev, cur in zip(eng.steps, eng.steps[1:]):
        if not cur[2]:
            assert set(cur[0]) <= set(prev[0])
    assert gen.generate(eng, prompts, max_tokens=0) == [[] for _ in prompts]


def test_stop_token_is_not_emitted_and_callback_sees_tokens(monkeypatch):
    monkeypatch.setattr(gen, "Sampler", FakeSampler)
    eng = FakeEngine()
    got = []
    outs = gen.generate(eng, [[3]], max_tokens=5, on_token=lambda r, t: got.append((r, t)))
    assert outs == [[]] and got == []                 # 3 mod 11 = 3 is the stop id
    outs = gen.generate(eng, [[1, 2], [5]], max_tokens=4, stop_ids=[], on_token=lambda r, t: got.append((r, t)))
    assert outs == [expected([1, 2], 4, ()), expected([5], 4, ())]
    assert [t for r, t in got if r == 0] == outs[0] and [t for r, t in got if r == 1] == outs[1]


def test_context_limit_ends_a_sequence(monkeypatch):
    monkeypatch.setattr(gen, "Sampler", FakeSampler)
    eng = FakeEngine()
    outs = gen.generate(eng, [[1] * 38], max_tokens=10, stop_ids=[])
    assert len(outs[0]) == 2 and eng.cache.live_slots() == []          # positions 38 and 39, then the limit


def test_kernel_error_words_are_read_at_the_end_of_every_batch_and_now_and_then(monkeypatch):
    eng = FakeEngine(max_tokens=PAGE_ROWS * 2)
    gen.generate(eng, [[1], [2], [3]], max_tokens=3, stop_ids=[], max_batch=1)
    assert eng.checks == [0, 0, 0]             # three batches of one: one look each, when the batch has ended
    monkeypatch.setattr(gen, "CHECK_EVERY", 2)
    eng = FakeEngine()
    gen.generate(eng, [[1]], max_tokens=7, stop_ids=[])
    assert eng.checks.count(1) >= 2 and eng.checks[-1] == 0

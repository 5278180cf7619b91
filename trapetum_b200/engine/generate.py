"""The generation loop: requests in, token ids out.

Requests are cut into batches that fit the cache; each batch starts together
(whole prompts of unequal lengths in one step), then every live sequence gets
one token per step.  A sequence ends at a stop id (which is not emitted,
runtime/src/bin/serve.rs:347-350), after ``max_tokens`` new tokens, or at the
model's context limit; its slot and pages go back at once and the batch
shrinks.  The next batch starts when the last sequence of this one has ended.
The reference's loop is one sequence, prompt token by token, then a fixed
number of greedy tokens (runtime/src/bin/gemma_run.rs:12-15).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..cache import pages_for
from ..csrc.ops import PAGE_ROWS
from ..sampling import Sampler, SamplingParams
from .engine import Engine
from .model import Model


CHECK_EVERY = 64          # decode steps between two looks at the kernels' error words (and at a batch's end)


def plan_batches(prompt_lens: Sequence[int], max_new: int, max_batch: int, max_tokens: int,
                 max_positions: int) -> List[List[int]]:
    """Cut requests, in order, into batches: at most ``max_batch`` sequences, and room in the cache
    for every sequence's prompt plus ``max_new`` tokens (counted in whole pages)."""
    if max_batch < 1:
        raise ValueError("max_batch must be at least 1")
    budget = pages_for(max_tokens)
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if n < 1:
            raise ValueError(f"request {i}: the prompt is empty")
        if n > max_positions:
            raise ValueError(f"request {i}: a prompt of {n} tokens exceeds the model's {max_positions} positions")
        need = pages_for(min(n + max_new, max_positions))
        if need > budget:
            raise ValueError(f"request {i}: {n} prompt tokens plus {max_new} new ones need {need * PAGE_ROWS} "
                             f"cache tokens, the cache holds {budget * PAGE_ROWS}")
        if cur and (len(cur) >= max_batch or used + need > budget):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


@dataclass
class _Seq:
    request: int
    slot: int
    length: int                  # tokens in the cache
    new: List[int] = field(default_factory=list)


def should_stop(token: int, n_new: int, length: int, stop_ids, max_new: int, max_positions: int) -> Optional[str]:
    """Why a sequence ends once ``token`` has been chosen as its next token, or None.
    ``n_new``: tokens emitted before this one; ``length``: tokens in the cache."""
    if token in stop_ids:
        return "stop"                       # the stop id itself is not emitted
    if n_new + 1 >= max_new:
        return "length"                     # this token is emitted and is the last
    if length + 1 > max_positions - 1:
        return "context"                    # it is emitted, but could not be followed by another
    return None


def generate(model_or_engine, prompts: Sequence[Sequence[int]], max_tokens: int = 256,
             temperature: float = 0.0, top_p: float = 0.95, repetition_penalty: float = 1.0, seed: int = 0,
             stop_ids: Optional[Sequence[int]] = None, max_batch: int = 64,
             cache_tokens: Optional[int] = None,
             on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
    """Generate up to ``max_tokens`` new ids for every prompt (lists of token ids).

    ``model_or_engine``: a loaded :class:`Model` (an engine is made for the call, its cache sized by
    ``cache_tokens`` or for one full batch) or an :class:`Engine` to reuse.  ``stop_ids``: None takes
    the model's ``eos_token_id``.  ``on_token(request, id)`` is called for each emitted token, like
    the reference's streaming callback (runtime/include/trapetum.h:20-27)."""
    params = SamplingParams(temperature=temperature, top_p=top_p, repetition_penalty=repetition_penalty,
                            max_tokens=max_tokens, seed=seed)
    prompts = [list(map(int, p)) for p in prompts]
    if hasattr(model_or_engine, "step") and hasattr(model_or_engine, "cache"):
        engine = model_or_engine
    else:
        model: Model = model_or_engine
        if cache_tokens is None:
            by_need = sorted((pages_for(min(len(p) + max_tokens, model.spec.max_positions)) for p in prompts),
                             reverse=True)
            cache_tokens = max(1, sum(by_need[:max_batch])) * PAGE_ROWS
        engine = Engine(model, cache_tokens, max_slots=max_batch)
    spec = engine.model.spec
    stops = frozenset(spec.stop_ids if stop_ids is None else stop_ids)
    outputs: List[List[int]] = [[] for _ in prompts]
    if max_tokens == 0 or not prompts:
        return outputs
    sampler = Sampler(params, engine.rt.device)
    greedy = not params.needs_sampler           # the engine then picks the token itself, on the device
    batches = plan_batches([len(p) for p in prompts], max_tokens, min(max_batch, engine.cache.max_slots),
                           engine.cache.max_tokens, spec.max_positions)
    for batch in batches:
        slots = engine.start(len(batch))
        live = [_Seq(r, s, 0) for r, s in zip(batch, slots)]
        steps = 0
        try:
            for q in live:
                sampler.begin(q.request, prompts[q.request])
            logits = engine.step([q.slot for q in live], [prompts[q.request] for q in live], borrow=True, greedy=greedy)
            for q in live:
                q.length = len(prompts[q.request])
            while live:
                chosen = sampler.choose(logits, [q.request for q in live])
                nxt: List[_Seq] = []
                for q, tok in zip(live, chosen):
                    why = should_stop(tok, len(q.new), q.length, stops, max_tokens, spec.max_positions)
                    if why != "stop":
                        q.new.append(tok)
                        if on_token is not None:
                            on_token(q.request, tok)
                    if why is None:
                        nxt.append(q)
                    else:
                        outputs[q.request] = q.new
                        sampler.end(q.request)
                        engine.release([q.slot])
                live = nxt
                if live:
                    logits = engine.step([q.slot for q in live], [[q.new[-1]] for q in live], borrow=True, greedy=greedy)
                    for q in live:
                        q.length += 1
                steps += 1
                if not live or steps % CHECK_EVERY == 0:
                    # the chosen tokens were just read on the host, so the device is idle anyway: a kernel whose
                    # bounded wait ran out must not pass its garbage on as tokens
                    engine.check_kernels()
        except BaseException:
            for q in live:
                if engine.cache.slots.is_held(q.slot):
                    engine.release([q.slot])
            raise
    return outputs

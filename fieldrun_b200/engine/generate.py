"""The generation loop above the step function.

Requests are taken in order into batches; a batch's prompts run in one step (in
several when together they pass ``PROMPT_TOKENS_PER_STEP``, a longer prompt in pieces, so that
a step's buffers stay bounded: a batch of 64 prompts of 2,048 tokens would otherwise need tens
of GB of them),
then every live sequence gets one token per step; a sequence that ends leaves
the following steps and gives its slot and pages back at once; the next batch
starts when the last sequence of this one has ended and uses the freed slots.  Per sequence the rules are the reference's stream loop
(src/minimax.rs:441-461): a stop token ends the sequence *before* it is put out,
the caller's ``emit`` may end it by returning False, and it ends at
``max_new_tokens``.  With ``ignore_eos`` it is the reference's fixed-length
``generate`` (src/minimax.rs:391-414), which checks no stop token.

The loop touches the engine only through ``new_sequence``, ``release``, ``step``
and ``pick`` and reads ``max_tokens``/``num_slots``; its decisions run on the host.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..cache import PAGE_TOKENS
from ..sampling import uniform


@dataclass(frozen=True)
class Request:
    prompt: tuple[int, ...]
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    eos: tuple[int, ...] = ()
    ignore_eos: bool = False
    index: int = 0                    # the request's number: names it to ``emit`` and keys its random numbers
    top_k: int = 0                    # sample among the k largest logits only (0: all)
    top_p: float = 1.0                # ... and among the smallest set of them that holds this much probability


@dataclass
class Generated:
    tokens: list[int] = field(default_factory=list)
    finish_reason: str = ""           # "eos" | "length" | "callback"


class GenerationError(ValueError):
    pass


PROMPT_TOKENS_PER_STEP = 16384      # most prompt tokens in one step


def prompt_steps(lengths: Sequence[int], budget: int) -> list[list[tuple[int, int, int]]]:
    """Cut a batch's prompts, in order, into steps of at most ``budget`` tokens.  A step is a list of pieces
    ``(position in lengths, first token, end token)``; a prompt longer than the budget is run in pieces of the
    budget, one step each (the cache keeps what the earlier pieces left, as in a decode step)."""
    steps: list[list[tuple[int, int, int]]] = []
    current: list[tuple[int, int, int]] = []
    held = 0
    for position, n in enumerate(lengths):
        if n > budget:
            if current:
                steps.append(current)
                current, held = [], 0
            steps.extend([[(position, first, min(first + budget, n))] for first in range(0, n, budget)])
            continue
        if current and held + n > budget:
            steps.append(current)
            current, held = [], 0
        current.append((position, 0, n))
        held += n
    if current:
        steps.append(current)
    return steps


def tokens_reserved(request: Request) -> int:
    """Cache tokens a request may come to hold, in whole pages.  The last generated token is never run."""
    most = len(request.prompt) + max(request.max_new_tokens - 1, 0)
    return (most + PAGE_TOKENS - 1) // PAGE_TOKENS * PAGE_TOKENS


def plan_batches(requests: Sequence[Request], *, max_batch: int, capacity_tokens: int, num_slots: int) -> list[list[int]]:
    """Cut the requests, in order, into batches that fit the cache.  Returns lists of positions in ``requests``."""
    if max_batch < 1:
        raise GenerationError(f"a batch size of {max_batch}")
    limit = min(max_batch, num_slots)
    batches: list[list[int]] = []
    current: list[int] = []
    held = 0
    for position, request in enumerate(requests):
        if not request.prompt:
            raise GenerationError(f"request {request.index} has an empty prompt")
        need = tokens_reserved(request)
        if need > capacity_tokens:
            raise GenerationError(
                f"request {request.index} may reach {need} tokens, the cache holds {capacity_tokens}")
        if current and (len(current) >= limit or held + need > capacity_tokens):
            batches.append(current)
            current, held = [], 0
        current.append(position)
        held += need
    if current:
        batches.append(current)
    return batches


def run_batch(engine, batch: Sequence[Request], emit: Optional[Callable[[int, int], Optional[bool]]] = None) -> list[Generated]:
    """Generate for requests that start together.  ``emit(request index, token)`` sees every token put out."""
    results = [Generated() for _ in batch]
    live = [b for b, r in enumerate(batch) if r.max_new_tokens > 0]
    for b, r in enumerate(batch):
        if r.max_new_tokens <= 0:
            results[b].finish_reason = "length"
    if not live:
        return results
    slots = {b: engine.new_sequence() for b in live}
    try:
        def pick(members, logits):
            temperatures = [batch[b].temperature for b in members]
            uniforms = [uniform(batch[b].seed, batch[b].index, len(results[b].tokens)) for b in members]
            if any(batch[b].top_k > 0 or batch[b].top_p < 1.0 for b in members):
                return engine.pick(logits, temperatures, uniforms, [batch[b].top_k for b in members],
                                   [batch[b].top_p for b in members])
            return engine.pick(logits, temperatures, uniforms)

        # the prompts: one step, or several when they are many tokens; the first tokens are picked step by step
        budget = getattr(engine, "prompt_tokens_per_step", PROMPT_TOKENS_PER_STEP)
        picked: list[int] = []
        for pieces in prompt_steps([len(batch[b].prompt) for b in live], budget):
            group = [live[i] for i, _, _ in pieces]
            ends = [end == len(batch[b].prompt) for b, (_, _, end) in zip(group, pieces)]
            logits = engine.step([slots[b] for b in group], [list(batch[b].prompt[first:end]) for b, (_, first, end) in zip(group, pieces)],
                                 [[end - first - 1] if last else [] for (_, first, end), last in zip(pieces, ends)])
            if all(ends):                                      # a piece that is not a prompt's last asks for no logits
                picked += pick(group, logits)
        logits = None
        while live:
            if logits is not None:
                picked = pick(live, logits)
            still: list[int] = []
            feed: list[list[int]] = []
            for b, token in zip(live, picked):
                request, result = batch[b], results[b]
                token = int(token)
                if not request.ignore_eos and token in request.eos:
                    result.finish_reason = "eos"              # the stop token is not put out
                    continue
                result.tokens.append(token)
                if emit is not None and emit(request.index, token) is False:
                    result.finish_reason = "callback"
                    continue
                if len(result.tokens) >= request.max_new_tokens:
                    result.finish_reason = "length"
                    continue
                still.append(b)
                feed.append([token])
            for b in live:
                if b not in still:
                    engine.release(slots.pop(b))              # an ended sequence holds nothing any longer
            live = still
            if live:
                logits = engine.step([slots[b] for b in live], feed)
    finally:
        for slot in slots.values():
            engine.release(slot)
    return results


def generate(engine, requests: Sequence[Request], *, max_batch: int = 64,
             emit: Optional[Callable[[int, int], Optional[bool]]] = None) -> list[Generated]:
    """Run every request, batch after batch; results come back in the order of ``requests``."""
    batches = plan_batches(requests, max_batch=max_batch, capacity_tokens=engine.max_tokens,
                           num_slots=engine.num_slots)
    results: list[Optional[Generated]] = [None] * len(requests)
    for positions in batches:
        for position, result in zip(positions, run_batch(engine, [requests[p] for p in positions], emit)):
            results[position] = result
    return [r for r in results if r is not None]

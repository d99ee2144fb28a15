"""The generation loop's decisions, with a scripted engine in place of the GPU."""
import numpy as np
import pytest

from fieldrun_b200.engine.generate import (GenerationError, Request, generate, plan_batches, prompt_steps, run_batch,
                                           tokens_reserved)
from fieldrun_b200.sampling import uniform


class ScriptedEngine:
    """The next token of a sequence is a function of its tokens so far: (sum + length) % vocab."""

    def __init__(self, vocab=50, max_tokens=4096, num_slots=8):
        self.vocab, self.max_tokens, self.num_slots = vocab, max_tokens, num_slots
        self.free = list(range(num_slots))[::-1]
        self.seqs = {}
        self.steps = []
        self.alloc_log = []
        self.release_log = []       # (slot, steps run when it was given back)

    def new_sequence(self):
        slot = self.free.pop()
        self.seqs[slot] = []
        self.alloc_log.append(slot)
        return slot

    def release(self, slot):
        assert slot in self.seqs, "released twice"
        del self.seqs[slot]
        self.free.append(slot)
        self.release_log.append((slot, len(self.steps)))

    def step(self, slots, tokens, want=None):
        assert len(set(slots)) == len(slots)
        self.steps.append([len(t) for t in tokens])
        rows = []
        for b, (slot, new) in enumerate(zip(slots, tokens)):
            self.seqs[slot].extend(new)
            if want is not None and list(want[b]) != [len(new) - 1]:
                assert list(want[b]) == []                   # the loop asks for the last place or for nothing
                continue
            nxt = (sum(self.seqs[slot]) + len(self.seqs[slot])) % self.vocab
            row = np.zeros(self.vocab, dtype=np.float32)
            row[nxt] = 5.0
            row[(nxt + 1) % self.vocab] = 4.0
            rows.append(row)
        return np.stack(rows) if rows else None

    def pick(self, logits, temperatures=None, uniforms=None, top_ks=None, top_ps=None):
        self.last_limits = (top_ks, top_ps)
        out = []
        for r, row in enumerate(logits):
            t = temperatures[r] if temperatures else 0.0
            if t > 0:
                p = np.exp((row - row.max()) / t)
                c = np.cumsum(p)
                out.append(int(np.searchsorted(c, uniforms[r] * c[-1], side="right")))
            else:
                out.append(int(np.argmax(row)))
        return out


def expected(prompt, n, vocab=50, eos=()):
    seq, out = list(prompt), []
    for _ in range(n):
        nxt = (sum(seq) + len(seq)) % vocab
        if nxt in eos:
            break
        out.append(nxt)
        seq.append(nxt)
    return out


def test_unequal_prompts_and_lengths_in_one_batch():
    engine = ScriptedEngine()
    reqs = [Request((1, 2, 3), 5, index=0), Request((4,), 2, index=1), Request((9, 9, 9, 9, 9, 9), 7, index=2)]
    results = run_batch(engine, reqs)
    assert [r.tokens for r in results] == [expected(r.prompt, r.max_new_tokens) for r in reqs]
    assert [r.finish_reason for r in results] == ["length"] * 3
    # prompts in one step, then one token each, shorter requests leaving: the last token is never run
    assert engine.steps == [[3, 1, 6], [1, 1, 1], [1, 1], [1, 1], [1, 1], [1], [1]]
    assert engine.seqs == {}


def test_stop_token_is_not_put_out_and_ends_only_its_sequence():
    engine = ScriptedEngine()
    prompt = (1, 2, 3)
    full = expected(prompt, 6)
    stop = full[2]
    reqs = [Request(prompt, 6, eos=(stop,), index=0), Request(prompt, 6, index=1),
            Request(prompt, 6, eos=(stop,), ignore_eos=True, index=2)]
    results = run_batch(engine, reqs)
    assert results[0].tokens == full[:2] and results[0].finish_reason == "eos"
    assert results[1].tokens == full and results[2].tokens == full
    assert results[2].finish_reason == "length"


def test_callback_can_end_a_sequence():
    engine = ScriptedEngine()
    seen = []

    def emit(index, token):
        seen.append((index, token))
        return False if (index == 1 and len([s for s in seen if s[0] == 1]) == 2) else None

    results = run_batch(engine, [Request((1,), 4, index=0), Request((2,), 4, index=1)], emit)
    assert len(results[0].tokens) == 4 and len(results[1].tokens) == 2
    assert results[1].finish_reason == "callback"
    assert [t for i, t in seen if i == 0] == results[0].tokens


def test_batches_one_after_another_reuse_slots():
    engine = ScriptedEngine(num_slots=2)
    reqs = [Request((i + 1, i + 2), 3 + i % 2, index=i) for i in range(5)]
    results = generate(engine, reqs, max_batch=8)
    assert [r.tokens for r in results] == [expected(r.prompt, r.max_new_tokens) for r in reqs]
    assert len(engine.alloc_log) == 5 and set(engine.alloc_log) == {0, 1}      # three batches through two slots
    assert engine.seqs == {} and sorted(engine.free) == [0, 1]


def test_plan_respects_batch_size_slots_and_cache():
    reqs = [Request(tuple(range(100)), 29, index=i) for i in range(5)]      # 128 reserved tokens each
    assert tokens_reserved(reqs[0]) == 128
    assert plan_batches(reqs, max_batch=2, capacity_tokens=10_000, num_slots=8) == [[0, 1], [2, 3], [4]]
    assert plan_batches(reqs, max_batch=8, capacity_tokens=10_000, num_slots=3) == [[0, 1, 2], [3, 4]]
    assert plan_batches(reqs, max_batch=8, capacity_tokens=300, num_slots=8) == [[0, 1], [2, 3], [4]]
    with pytest.raises(GenerationError, match="cache holds"):
        plan_batches(reqs, max_batch=8, capacity_tokens=64, num_slots=8)
    with pytest.raises(GenerationError, match="empty prompt"):
        plan_batches([Request((), 3)], max_batch=1, capacity_tokens=64, num_slots=1)


def test_zero_new_tokens_runs_nothing():
    engine = ScriptedEngine()
    results = run_batch(engine, [Request((1, 2), 0)])
    assert results[0].tokens == [] and results[0].finish_reason == "length" and engine.steps == []


def test_slots_come_back_when_a_step_fails():
    engine = ScriptedEngine()

    def boom(*a, **k):
        raise RuntimeError("step failed")

    engine.step = boom
    with pytest.raises(RuntimeError):
        run_batch(engine, [Request((1,), 3)])
    assert engine.seqs == {}


def test_uniform_numbers_depend_only_on_seed_request_and_step():
    values = {(s, r, n): uniform(s, r, n) for s in (0, 1) for r in (0, 1, 7) for n in range(4)}
    assert all(0.0 <= v < 1.0 for v in values.values())
    assert len(set(values.values())) == len(values)
    assert uniform(3, 4, 5) == uniform(3, 4, 5)
    assert np.float32(uniform(9, 9, 9)) == uniform(9, 9, 9)           # exact in float32
    many = [uniform(0, 0, n) for n in range(4000)]
    assert 0.45 < np.mean(many) < 0.55


def test_sampling_is_per_request_not_per_batch_position():
    reqs = [Request((i + 1,), 6, temperature=1.5, seed=3, index=i) for i in range(4)]
    together = generate(ScriptedEngine(), reqs, max_batch=4)
    alone = [generate(ScriptedEngine(), [r], max_batch=1)[0] for r in reqs]
    assert [r.tokens for r in together] == [r.tokens for r in alone]
    other_seed = generate(ScriptedEngine(), [Request(r.prompt, 6, 1.5, 4, index=r.index) for r in reqs])
    assert [r.tokens for r in other_seed] != [r.tokens for r in together]


def test_many_prompt_tokens_are_run_in_several_steps():
    assert prompt_steps([5, 5, 5], 10) == [[(0, 0, 5), (1, 0, 5)], [(2, 0, 5)]]
    assert prompt_steps([25, 1, 1], 10) == [[(0, 0, 10)], [(0, 10, 20)], [(0, 20, 25)], [(1, 0, 1), (2, 0, 1)]]   # a long prompt in pieces
    assert prompt_steps([3], 10) == [[(0, 0, 3)]]
    engine = ScriptedEngine()
    engine.prompt_tokens_per_step = 10
    prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11], [12, 13], [14] * 23]
    requests = [Request(tuple(p), 4, index=i) for i, p in enumerate(prompts)]
    results = run_batch(engine, requests)
    assert engine.steps[:5] == [[6], [5, 2], [10], [10], [3]]     # five prompt steps, then all four decode together
    assert engine.steps[5] == [1, 1, 1, 1]
    for p, r in zip(prompts, results):
        assert r.tokens == expected(p, 4)


def test_top_k_and_top_p_reach_the_pick():
    engine = ScriptedEngine()
    requests = [Request((1, 2), 2, temperature=0.7, seed=3, index=0, top_k=5, top_p=0.9), Request((3,), 2, temperature=0.7, index=1)]
    run_batch(engine, requests)
    assert engine.last_limits == ([5, 0], [0.9, 1.0])
    run_batch(engine, [Request((1, 2), 2, temperature=0.7, index=0)])
    assert engine.last_limits == (None, None)                      # nothing to cut: the plain call


def test_an_ended_sequence_gives_its_slot_back_at_once():
    engine = ScriptedEngine()
    reqs = [Request((1, 2, 3), 5, index=0), Request((4,), 2, index=1), Request((9, 9), 7, index=2)]
    run_batch(engine, reqs)
    # slots 0, 1, 2 in the order of the requests; request 1 ends after 2 steps, request 0 after 5, request 2 after 7
    assert engine.release_log == [(1, 2), (0, 5), (2, 7)]
    assert engine.seqs == {} and sorted(engine.free) == list(range(8))

"""The engine against the plain implementation, in float32 and in bfloat16: whole requests, the last
tokens one by one, batches of unequal lengths through few slots, long decoding, the first tokens."""
import numpy as np
import pytest
import torch

import plain_model as pm
from gpu_helpers import (TOLERANCE, RouteRecorder, assert_close, check_request, loaded, model_folder, plain_logits,
                         plain_margins, plain_weights, request_tokens, run_schedule, worst)
from tiny_configs import ALL

pytestmark = pytest.mark.gpu

NAMES = list(ALL)
DTYPES = ["float32", "bfloat16"]
LENGTHS = [1, 5, 13, 40, 64, 77, 130]


def to_np(t):
    return t.float().cpu().numpy()


def run_and_check(name, dtype, lm, requests, steps, what):
    """Runs the schedule and compares every request with the plain model (see gpu_helpers.check_request)."""
    if dtype == "bfloat16":
        with RouteRecorder(lm) as recorder:
            logits = run_schedule(lm, requests, steps, recorder)
        for key, ids in requests.items():
            check_request(name, dtype, ids, logits[key], recorder.of(key, len(ids)), f"{name} {what}, request {key}")
    else:
        logits = run_schedule(lm, requests, steps)
        for key, ids in requests.items():
            check_request(name, dtype, ids, logits[key], None, f"{name} {what}, request {key}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(name, dtype):
    lm = loaded(name, dtype)
    requests = {n: request_tokens(name, n, 0) for n in LENGTHS + [300]}
    run_and_check(name, dtype, lm, requests, [[(n, 0, n)] for n in requests], "whole")
    assert lm.engine.cache.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(name, dtype):
    lm = loaded(name, dtype)
    requests = {n: request_tokens(name, n, 0) for n in (40, 77, 130)}
    steps = []
    for n in requests:
        steps.append([(n, 0, n - 32)])
        steps.extend([[(n, j, j + 1)] for j in range(n - 32, n)])
    run_and_check(name, dtype, lm, requests, steps, "last 32 one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_through_few_slots(name, dtype):
    """Three slots, seven requests: prompts of a batch in one step, then one token each, the shorter
    ones leaving earlier; the next batch takes the freed slots."""
    lm = loaded(name, dtype, 2048, 3)
    plan = [(130, 9), (5, 2), (77, 20), (1, 0), (64, 33), (40, 39), (13, 5)]      # (length, decoded at the end)
    requests = {n: request_tokens(name, n, 0) for n, _ in plan}
    steps = []
    for start in range(0, len(plan), 3):
        batch = plan[start:start + 3]
        steps.append([(n, 0, n - dec) for n, dec in batch])
        for k in range(max(dec for _, dec in batch)):
            steps.append([(n, n - dec + k, n - dec + k + 1) for n, dec in batch if k < dec])
    run_and_check(name, dtype, lm, requests, steps, "unequal batches")
    assert lm.engine.cache.slots.num_held == 0


@pytest.mark.parametrize("name", ["a", "d"])
def test_recorded_steps_in_bfloat16(name):
    """The same decode steps replayed from their recording and run directly: the same logits, bit for bit."""
    lm = loaded(name, "bfloat16")
    requests = {n: request_tokens(name, n, 5) for n in (70, 9, 33)}
    steps = [[(n, 0, n - 8) for n in requests]] + [[(n, n - 8 + k, n - 7 + k) for n in requests] for k in range(8)]
    lm.engine.record_steps = True
    before = lm.engine.steps_replayed
    replayed = run_schedule(lm, requests, steps)
    assert lm.engine.steps_replayed >= before + 6
    lm.engine.record_steps = False
    try:
        direct = run_schedule(lm, requests, steps)
    finally:
        lm.engine.record_steps = True
    for n in requests:
        np.testing.assert_array_equal(replayed[n], direct[n])


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(dtype):
    name = "a"
    lm = loaded(name, dtype)
    engine = lm.engine
    length = 230
    ids = request_tokens(name, length, 3)
    ref = plain_logits(name, length, 3)
    slot = engine.new_sequence()
    try:
        rows = [to_np(engine.step([slot], [[t]], [[0]])) for t in ids]       # from the very first token
    finally:
        engine.release(slot)
    got = np.concatenate(rows)
    assert_close(got[:3], ref[:3], dtype, "the first tokens", plain_margins(name, length, 3)[:3])
    assert_close(got, ref, dtype, "230 tokens one by one", plain_margins(name, length, 3))


@pytest.mark.parametrize("name", NAMES)
def test_padding_and_company_change_nothing(name):
    """The same request alone, and beside others of other lengths, in float32: the same logits up to rounding."""
    lm = loaded(name, "float32")
    engine = lm.engine
    ids = request_tokens(name, 40, 0)
    alone = to_np(lm.logits(ids))
    others = [request_tokens(name, n, 1) for n in (3, 90)]
    slots = [engine.new_sequence() for _ in range(3)]
    try:
        out = to_np(engine.step(slots, [others[0], ids, others[1]], [[], list(range(40)), []]))
    finally:
        for s in slots:
            engine.release(s)
    assert worst(out, alone) < 2e-6


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(name):
    lm = loaded(name, "float32")
    config, weights = plain_weights(name)
    prompt = request_tokens(name, 9, 2)
    want = pm.generate_greedy(config, weights, prompt, 12)
    assert lm.generate(prompt, 12) == want
    assert lm.predict(prompt) == want[0]
    stop = want[4]
    cut = want[:want.index(stop)]
    assert lm.generate_stream(prompt, 12, eos=[stop]) == cut
    seen = []
    assert lm.generate_stream(prompt, 12, emit=lambda t: (seen.append(t), len(seen) < 3)[1]) == want[:3]
    prompts = [request_tokens(name, n, 2) for n in (9, 2, 30, 17)]
    outs, reasons = lm.generate_batch(prompts, 6, eos=[], return_reasons=True)
    assert outs == [pm.generate_greedy(config, weights, p, 6) for p in prompts] and reasons == ["length"] * 4
    lm.engine.cache.check()
    assert lm.engine.cache.slots.num_held == 0


def test_greedy_generation_in_bfloat16_stays_on_the_plain_models_top():
    name = "b"
    lm = loaded(name, "bfloat16")
    config, weights = plain_weights(name)
    prompt = request_tokens(name, 20, 2)
    out = lm.generate(prompt, 16)
    ref = pm.logits_all_positions(config, weights, prompt + out)
    for i, token in enumerate(out):
        row = ref[len(prompt) - 1 + i]
        assert row[token] >= row.max() - 2 * TOLERANCE["bfloat16"] * np.abs(ref).max()


def test_prompts_in_pieces_generate_what_whole_prompts_do():
    """With a budget of 20 prompt tokens a step, prompts of 6 to 70 tokens run as whole prompts sharing steps and
    as pieces of 20: the same tokens as with every prompt whole in one step."""
    name = "b"
    lm = loaded(name, "float32")
    prompts = [request_tokens(name, n, 7) for n in (6, 70, 9, 45, 20)]
    whole = lm.generate_batch(prompts, 6, eos=[])
    budget = lm.engine.prompt_tokens_per_step
    lm.engine.prompt_tokens_per_step = 20
    try:
        assert lm.generate_batch(prompts, 6, eos=[]) == whole
    finally:
        lm.engine.prompt_tokens_per_step = budget


def test_temperature_sampling_repeats_with_its_seed_and_follows_the_plain_pick():
    from fieldrun_b200.sampling import uniform
    name = "a"
    lm = loaded(name, "float32")
    config, weights = plain_weights(name)
    prompts = [request_tokens(name, n, 4) for n in (6, 11)]
    first = lm.generate_batch(prompts, 10, eos=[], temperature=0.8, seed=5)
    assert first == lm.generate_batch(prompts, 10, eos=[], temperature=0.8, seed=5)
    assert first != lm.generate_batch(prompts, 10, eos=[], temperature=0.8, seed=6)
    for index, (prompt, out) in enumerate(zip(prompts, first)):
        seq = list(prompt)
        for step, token in enumerate(out):
            row = pm.logits_all_positions(config, weights, seq)[-1]
            assert token == pm.temperature_pick(row, 0.8, uniform(5, index, step))
            seq.append(token)
    # with only the largest logit kept, sampling is the greedy pick; with limits it follows the plain pick among the kept
    assert lm.generate_batch(prompts, 6, eos=[], temperature=0.8, seed=5, top_k=1) == lm.generate_batch(prompts, 6, eos=[])
    limited = lm.generate_batch(prompts, 8, eos=[], temperature=1.5, seed=9, top_k=12, top_p=0.7)
    for index, (prompt, out) in enumerate(zip(prompts, limited)):
        seq = list(prompt)
        for step, token in enumerate(out):
            row = pm.logits_all_positions(config, weights, seq)[-1]
            assert token == pm.top_k_top_p_pick(row, 1.5, uniform(9, index, step), 12, 0.7)
            seq.append(token)
    with pytest.raises(ValueError):
        lm.generate_batch(prompts, 2, temperature=0.8, top_p=0.0)


def test_errors_come_before_any_launch():
    from fieldrun_b200.cache import CacheFull
    from fieldrun_b200.engine import StepError
    lm = loaded("a", "float32", 2048, 3)
    engine = lm.engine
    slot = engine.new_sequence()
    try:
        with pytest.raises(StepError, match="outside the vocabulary"):
            engine.step([slot], [[1, 256]])
        with pytest.raises(StepError, match="wanted place"):
            engine.step([slot], [[1, 2]], [[2]])
        with pytest.raises(StepError, match="position tables end"):
            engine.step([slot], [[1] * 2049])
        other = engine.new_sequence()
        with pytest.raises(CacheFull, match="pages"):
            engine.step([slot, other], [[1] * 1500, [2] * 600])
        engine.release(other)
        assert engine.length(slot) == 0
        assert engine.step([slot], [[1, 2, 3]], [[]]) is None and engine.length(slot) == 3
    finally:
        engine.release(slot)
    engine.cache.check()


def test_a_long_request_over_many_pages_and_key_chunks():
    """2,500 tokens as a prompt, then 60 more one by one: forty pages, ten key chunks per decode step, the
    chunks' partial results merged in order."""
    name, dtype = "b", "bfloat16"
    lm = loaded(name, dtype, 4096, 2)
    n = 2560
    requests = {"long": request_tokens(name, n, 9)}
    steps = [[("long", 0, 2500)]] + [[("long", j, j + 1)] for j in range(2500, n)]
    with RouteRecorder(lm) as recorder:
        logits = run_schedule(lm, requests, steps, recorder)
    # the plain model on 2,560 tokens is slow: compare the prompt's last rows and every decoded row
    config, weights = plain_weights(name)
    sizes = pm.sizes_from_config(config)
    hidden = pm.hidden_states(config, weights, requests["long"], forced_routes=recorder.of("long", n))
    ref = hidden[2400:] @ weights["lm_head.weight"].astype(np.float64).T
    assert_close(logits["long"][2400:], ref, dtype, "a request of 2,560 tokens")
    assert sizes["layers"] == 3


M2_SHAPED = dict(
    architectures=["MiniMaxM2ForCausalLM"], model_type="minimax_m2", num_hidden_layers=1, hidden_size=3072,
    num_attention_heads=48, num_key_value_heads=8, head_dim=128, rotary_dim=64, rope_theta=5000000.0, use_qk_norm=True,
    num_local_experts=16, num_experts_per_tok=8, intermediate_size=1536, vocab_size=2003, rms_norm_eps=1e-6,
    tie_word_embeddings=False)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_a_layer_of_minimax_m2_size(dtype):
    """One layer with MiniMax-M2's own sizes (48 heads over 8, head size 128 with 64 rotary dims, q/k norms
    6,144 and 1,024 wide, experts 3,072 x 1,536, top 8; fewer experts and a small vocabulary keep the folder
    small): a prompt long enough for the tcgen05 kernels, then decode steps on the streaming kernels; in
    float32 the same through the general kernels."""
    import tempfile

    import fieldrun_b200 as fr
    with tempfile.TemporaryDirectory() as folder:
        fr.write_random_model(folder, M2_SHAPED, fr.RandomInit(seed=4, matrix_std=0.02, norm_std=0.1, bias_std=0.01))
        config, weights = pm.read_model_folder(folder)
        lm = fr.load(folder, dtype=dtype, max_tokens=512)
        ids = np.random.default_rng(11).integers(0, 2003, size=76).tolist()
        requests = {"r": ids, "s": ids[5:30]}
        steps = [[("r", 0, 70), ("s", 0, 20)]] + [[("r", 70 + k, 71 + k)] + ([("s", 20 + k, 21 + k)] if k < 5 else []) for k in range(6)]
        with RouteRecorder(lm) as recorder:
            logits = run_schedule(lm, requests, steps, recorder)
        for key, tokens in requests.items():
            routes = recorder.of(key, len(tokens))
            hidden, margins, own = pm.hidden_states(config, weights, tokens, forced_routes=routes, return_routes=True)
            ref = hidden @ weights["lm_head.weight"].astype(np.float64).T
            assert_close(logits[key], ref, dtype, f"MiniMax-M2-sized layer, request {key}")
            differs = (np.sort(own, axis=-1) != np.sort(routes, axis=-1)).any(axis=-1)
            assert not (differs & (margins > (5e-3 if dtype == "bfloat16" else 1e-5))).any()


def test_a_step_whose_buffers_pass_two_to_the_31_elements():
    """A prompt of 95,000 tokens beside a short one, one layer of MiniMax-M2's own sizes: the expert outputs of
    the step are 760,000 rows of 3,072 float32, more elements than 32-bit indices reach, and the short
    request's rows lie at the far end of every buffer.  Its logits must be what it gets alone (no plain
    model at this size: an index that wrapped would read or write some other row)."""
    import fieldrun_b200 as fr
    lm = fr.random_model(M2_SHAPED, fr.RandomInit(seed=4, matrix_std=0.02, norm_std=0.1, bias_std=0.01), dtype="bfloat16",
                         max_tokens=96 * 1024, num_slots=2)
    engine = lm.engine
    rng = np.random.default_rng(12)
    long_ids = rng.integers(0, 2003, size=95_000).tolist()
    short_ids = rng.integers(0, 2003, size=200).tolist()
    slot = engine.new_sequence()
    alone = engine.step([slot], [short_ids], [[0, 100, 199]]).float().cpu().numpy()
    engine.release(slot)
    slots = [engine.new_sequence(), engine.new_sequence()]
    both = engine.step(slots, [long_ids, short_ids], [[94_999], [0, 100, 199]]).float().cpu().numpy()
    assert np.isfinite(both).all()
    err = np.abs(both[1:] - alone).max() / np.abs(alone).max()
    assert err <= TOLERANCE["bfloat16"], f"the short request beside a long one: relative difference {err:.3e}"
    after = engine.step(slots, [[5], [7]]).float().cpu().numpy()          # one more token each, over the long cache
    assert np.isfinite(after).all()
    for s_ in slots:
        engine.release(s_)
    engine.cache.check()


def test_a_kernel_that_gave_up_stops_the_generation_loop():
    """The status word, set by a kernel whose wait ran out (here by the probe whose wait is meant to), reaches
    the host with the next picked tokens and ends the run with an error instead of tokens."""
    from fieldrun_b200.csrc import ops
    lm = loaded("a", "bfloat16")
    ops.wait_probe(lm.engine.device, limit_cycles=50_000)
    with pytest.raises(ops.KernelError, match="gave up"):
        lm.generate([1, 2, 3], 4)
    assert lm.engine.cache.slots.num_held == 0                   # the loop gave its slot back on the way out
    assert len(lm.generate([1, 2, 3], 4)) == 4                   # and the next run is clean
    ops.wait_probe(lm.engine.device, limit_cycles=50_000)
    with pytest.raises(ops.KernelError, match="gave up"):
        lm.logits([1, 2, 3])
    lm.engine.check()


# --------------------------------------------------------------------------- schedules beyond the three cuttings

@pytest.mark.parametrize("name", ["d", "b"])
def test_prompts_in_pieces_and_steps_that_mix_pieces_with_single_tokens(name):
    """bfloat16, logits against the plain model with the engine's picks forced.  Configuration d has the sizes
    the tcgen05 kernels take, so a prompt piece of 64 or more tokens that starts beyond position 0 runs on them
    inside the engine.  The steps: a long prompt in three pieces; then a step that holds a piece of a second
    prompt, a whole short prompt and a single token of the first request together; then single tokens beside the
    second prompt's next piece."""
    dtype = "bfloat16"
    lm = loaded(name, dtype)
    requests = {"long": request_tokens(name, 330, 21), "second": request_tokens(name, 200, 22),
                "short": request_tokens(name, 11, 23)}
    steps = [
        [("long", 0, 100)],
        [("long", 100, 228)],                                    # 128 tokens at position 100
        [("long", 228, 320)],
        [("second", 0, 70), ("short", 0, 9), ("long", 320, 321)],  # a piece, a whole short prompt, one token
        [("second", 70, 198), ("short", 9, 10), ("long", 321, 322)],
        [("long", 322, 323), ("second", 198, 199), ("short", 10, 11)],
    ] + [[("long", j, j + 1)] + ([("second", 199, 200)] if j == 323 else []) for j in range(323, 330)]
    run_and_check(name, dtype, lm, requests, steps, "pieces and mixed steps")
    assert lm.engine.cache.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompts_in_pieces_in_float32_and_bfloat16_at_every_configuration(dtype):
    for name in NAMES:
        lm = loaded(name, dtype)
        requests = {"r": request_tokens(name, 150, 31)}
        run_and_check(name, dtype, lm, requests, [[("r", 0, 64)], [("r", 64, 141)], [("r", 141, 150)]], "a prompt in pieces")


def test_recorded_steps_across_a_length_range_and_past_the_number_kept(monkeypatch):
    """bfloat16 with recording on, against the plain model: decoding from length 1,000 to 1,050 leaves the
    recording for lengths up to 1,024 and enters the next one (other chunk counts in the attention); then more
    batch sizes than recordings are kept, and the first size again after it was dropped."""
    from fieldrun_b200.engine import engine as engine_module
    name, dtype = "d", "bfloat16"
    lm = loaded(name, dtype, 4096, 8)
    engine = lm.engine
    assert engine.record_steps
    n = 1050
    requests = {"r": request_tokens(name, n, 41)}
    steps = [[("r", 0, 1000)]] + [[("r", j, j + 1)] for j in range(1000, n)]
    with RouteRecorder(lm) as recorder:
        recorded_before, replayed_before = engine.steps_recorded, engine.steps_replayed
        logits = run_schedule(lm, requests, steps, recorder)
        assert engine.steps_recorded == recorded_before + 2           # lengths up to 1,024, then up to 2,048
        assert engine.steps_replayed == replayed_before + 48
        config, weights = plain_weights(name)
        hidden = pm.hidden_states(config, weights, requests["r"], forced_routes=recorder.of("r", n))
        ref = hidden[990:] @ weights["lm_head.weight"].astype(np.float64).T
        assert_close(logits["r"][990:], ref, dtype, "decoding across a recording's length range")

    monkeypatch.setattr(engine_module, "RECORDED_STEPS_KEPT", 3)
    engine._recorded.clear()
    sizes = [1, 2, 3, 4, 6, 1]                                        # six sizes through three kept recordings
    prompts = [request_tokens(name, 5 + b, 42) for b in range(6)]
    config, weights = plain_weights(name)

    def run(record):
        engine.record_steps = record
        out = []
        for size in sizes:
            slots = [engine.new_sequence() for _ in range(size)]
            engine.step(slots, [p[:-2] for p in prompts[:size]], [[] for _ in range(size)])
            out.append(engine.step(slots, [[p[-2]] for p in prompts[:size]]).float().cpu().numpy())
            out.append(engine.step(slots, [[p[-1]] for p in prompts[:size]]).float().cpu().numpy())
            for s in slots:
                engine.release(s)
        return out

    before = engine.steps_recorded
    replayed = run(True)
    assert engine.steps_recorded == before + 6 and len(engine._recorded) == 3    # size 1 was dropped and made again
    direct = run(False)
    engine.record_steps = True
    for a, b in zip(replayed, direct):
        np.testing.assert_array_equal(a, b)
    for size, rows in zip(sizes, replayed[1::2]):
        for b in range(size):
            if plain_margins(name, 5 + b, 42).min() < 5e-3:          # a near tie of the router may go either way
                continue
            ref = plain_logits(name, 5 + b, 42)[-1]
            assert np.abs(rows[b] - ref).max() <= TOLERANCE[dtype] * np.abs(plain_logits(name, 5 + b, 42)).max()


def test_sixteen_requests_that_all_end_at_different_steps():
    """generate_batch in float32 with sixteen prompts and sixteen different stop tokens' worth of lengths: the
    tokens are the plain model's, every sequence's slot and pages go back the moment it ends, and a batch that
    shrinks from sixteen to one runs through a handful of recordings, not one per size."""
    name = "a"
    lm = loaded(name, "float32", 4096, 16)
    engine = lm.engine
    config, weights = plain_weights(name)
    prompts = [request_tokens(name, 3 + 2 * i, 51) for i in range(16)]
    lengths = [2 + i for i in range(16)]                              # all different
    from fieldrun_b200.engine.generate import Request, generate
    requests = [Request(tuple(p), n, ignore_eos=True, index=i) for i, (p, n) in enumerate(zip(prompts, lengths))]
    engine._recorded.clear()
    before = engine.steps_recorded
    held = []
    results = generate(engine, requests, max_batch=16, emit=lambda i, t: held.append(engine.cache.slots.num_held))
    for p, n, r in zip(prompts, lengths, results):
        assert r.tokens == pm.generate_greedy(config, weights, p, n) and r.finish_reason == "length"
    assert engine.steps_recorded - before <= 8                       # 16, 12, 8, 6, 4, 3, 2, 1
    assert max(held) == 16 and min(held) == 1 and engine.cache.slots.num_held == 0
    engine.cache.check()


@pytest.mark.parametrize("name", ["a", "d"])
def test_company_in_the_batch_changes_bfloat16_logits_by_rounding_only(name):
    """The same request alone and beside others of other lengths, as a prompt and then token by token, in
    bfloat16.  What differs is the order of partial sums (how many parts an inner size or a sequence's keys are
    cut into follows the step's shape): float32 rounding of a sum of bfloat16 products, far below the distance to
    the plain model.  A router choice that such rounding tips would show as a jump; the bound excludes it."""
    lm = loaded(name, "bfloat16")
    engine = lm.engine
    ids = request_tokens(name, 48, 0)
    others = [request_tokens(name, n, 1) for n in (3, 90)]

    def run(with_company):
        slots = [engine.new_sequence() for _ in range(3 if with_company else 1)]
        try:
            if with_company:
                out = [to_np(engine.step(slots, [others[0][:2], ids[:40], others[1][:80]], [[], list(range(40)), []]))]
                for k in range(8):
                    live = slots if k < 1 else slots[1:]
                    feed = [[others[0][2]]] * (k < 1) + [[ids[40 + k]], [others[1][80 + k]]]
                    out.append(to_np(engine.step(live, feed))[len(live) - 2:len(live) - 1])
            else:
                out = [to_np(engine.step(slots, [ids[:40]], [list(range(40))]))]
                out += [to_np(engine.step(slots, [[ids[40 + k]]])) for k in range(8)]
        finally:
            for s in slots:
                engine.release(s)
        return np.concatenate(out)

    alone, beside = run(False), run(True)
    # measured on a B200: 0 at configuration a, 1.5e-7 at configuration d
    assert worst(beside, alone) < 1e-5, f"relative difference {worst(beside, alone):.2e}"
    assert worst(alone, plain_logits(name, 48, 0)) < TOLERANCE["bfloat16"] * 4


def test_what_an_earlier_request_left_in_the_cache_reaches_no_later_one():
    """Every page of the store is filled with NaN before any request runs, as if earlier requests had left
    non-finite keys and values everywhere, the tails of their last pages included.  The requests that follow
    must compute what they compute on a clean store, bit for bit: a page is cleared when it is handed out."""
    for dtype in DTYPES:
        name = "d" if dtype == "bfloat16" else "b"
        import fieldrun_b200 as fr
        lm = fr.load(model_folder(name), dtype=dtype, max_tokens=1024, num_slots=3)
        engine = lm.engine
        requests = {n: request_tokens(name, n, 61) for n in (70, 9, 130)}
        steps = [[(n, 0, n - 8) for n in requests]] + [[(n, n - 8 + k, n - 7 + k) for n in requests] for k in range(8)]
        clean = run_schedule(lm, requests, steps)
        for group in engine.cache.groups:
            group.keys.fill_(float("nan"))
            group.values.fill_(float("nan"))
        poisoned = run_schedule(lm, requests, steps)
        for n in requests:
            assert np.isfinite(poisoned[n]).all(), f"{dtype}: NaN left in the cache reached request {n}"
            np.testing.assert_array_equal(poisoned[n], clean[n])


def test_the_reference_gates_own_form_sixty_windows_of_sixteen_tokens():
    """The reference validates this architecture by top-1 agreement on 60 sliding windows: for i in 16..76 the
    model sees ids[i-16:i] from position 0 and predicts the next token (scripts/gemma3_ref.py:250-262,
    scripts/validate_all.sh:28-29: --ctx 16 --n-eval 60, 60/60 required in float32), on a tiny model whose norm
    weights are drawn around zero and whose routing bias is drawn wide (gemma3_ref.py:223-247).  Configuration e
    is that model's config.json as its writer emits it, with weights by that recipe."""
    name = "e"
    config, weights = plain_weights(name)
    ids = request_tokens(name, 76, 71)
    want = [pm.greedy_pick(pm.logits_all_positions(config, weights, ids[i - 16:i])[-1]) for i in range(16, 76)]
    lm = loaded(name, "float32")
    got = [lm.predict(ids[i - 16:i]) for i in range(16, 76)]
    assert got == want                                              # 60 of 60
    # in bfloat16 the same windows, each pick held to the plain model's top within the tolerance
    lm16 = loaded(name, "bfloat16")
    agree = 0
    for i in range(16, 76):
        row = pm.logits_all_positions(config, weights, ids[i - 16:i])[-1]
        pick = lm16.predict(ids[i - 16:i])
        agree += pick == want[i - 16]
        assert row[pick] >= row.max() - 2 * TOLERANCE["bfloat16"] * np.abs(row).max()
    assert agree >= 57, f"bfloat16 agrees with the plain model on {agree} of 60 windows"      # measured: 60


def test_random_weights_are_the_same_bits_on_the_device_and_on_the_host():
    """A model drawn on the device (fr.random_model, what the benchmark runs) and the folder written on the host
    from the same configuration and seed hold the same weights, so a model too large to write can still be
    re-made, tensor by tensor, for the plain implementation."""
    import fieldrun_b200 as fr
    from fieldrun_b200.weights import TensorNeed
    config, init = ALL["b"]
    _, weights = plain_weights("b")
    drawn = fr.random_model(config, init, dtype="float32", max_tokens=128)
    loaded_from_folder = loaded("b", "float32")
    for a, b in zip(drawn.model.all_parts(), loaded_from_folder.model.all_parts()):
        for key, value in vars(a).items():
            if isinstance(value, torch.Tensor) and value.is_floating_point() and key not in ("cos", "sin"):
                assert torch.equal(value, getattr(b, key)), f"{type(a).__name__}.{key}"
    name = "model.layers.1.block_sparse_moe.experts.3.w2.weight"
    on_device = init.draw(TensorNeed(name, weights[name].shape), "cuda").float().cpu().numpy()
    np.testing.assert_array_equal(on_device, weights[name])
    ids = request_tokens("b", 20, 81)
    np.testing.assert_array_equal(to_np(drawn.logits(ids)), to_np(loaded_from_folder.logits(ids)))


def test_positions_beyond_sixty_thousand_against_the_plain_model():
    """One layer of configuration a's sizes, a sequence of 65,536 tokens in float32: the logits of the last
    positions of the prompt and of decoded tokens at positions 65,500 to 65,535 against the plain model, which
    computes those rows only (the square of scores of the whole sequence would not fit).  Rotary angles there
    are tens of thousands of radians in the fast pairs; the tables hold them exactly (see the table test)."""
    import fieldrun_b200 as fr
    from tiny_configs import CONFIG_A, INIT_A
    config = {**CONFIG_A, "num_hidden_layers": 1, "rope_theta": 5000000.0}
    lm = fr.random_model(config, INIT_A, dtype="float32", max_tokens=65536, num_slots=1)
    from fieldrun_b200.weights import TensorNeed
    needs = {n.name: n for n in lm.model.tensor_needs()}
    W = {name: INIT_A.draw(need, "cuda").double().cpu().numpy() for name, need in needs.items()}
    s = pm.sizes_from_config(config)
    n, tail = 65536, 40
    ids = np.random.default_rng(91).integers(0, s["vocab"], size=n)
    rows = np.arange(n - tail, n)
    x = W["model.embed_tokens.weight"][ids]
    p = "model.layers.0."
    a = pm.rms_norm(x, W[p + "input_layernorm.weight"], s["eps"])
    x_tail = x[rows] + pm.attention_layer(a, W, p, s, np.arange(n), rows=rows)
    a2 = pm.rms_norm(x_tail, W[p + "post_attention_layernorm.weight"], s["eps"])
    y, margin = pm.routed_experts(a2, W, p, s)
    ref = pm.rms_norm(x_tail + y, W["model.norm.weight"], s["eps"]) @ W["lm_head.weight"].T
    engine = lm.engine
    slot = engine.new_sequence()
    prompt_end = n - 36
    got = [to_np(engine.step([slot], [ids[:prompt_end].tolist()], [list(range(prompt_end - 4, prompt_end))]))]
    got += [to_np(engine.step([slot], [[int(ids[j])]])) for j in range(prompt_end, n)]
    engine.release(slot)
    got = np.concatenate(got)
    clear = margin > 1e-5
    assert clear.sum() >= tail - 2
    assert_close(got[clear], ref[clear], "float32", "positions 65,496 to 65,535")

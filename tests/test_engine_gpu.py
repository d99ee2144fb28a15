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

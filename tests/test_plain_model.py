"""The plain implementation checked against the reference's formulas written out element by element."""
import math

import numpy as np
import pytest

import fieldrun_b200 as fr
import plain_model as pm
from tiny_configs import ALL


def test_rms_norm_elementwise():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(3, 10)), rng.normal(size=10)
    out = pm.rms_norm(x, w, 1e-5)
    for r in range(3):
        ms = sum(v * v for v in x[r]) / 10                      # src/minimax.rs:61-62
        for i in range(10):
            assert out[r, i] == pytest.approx(x[r, i] * (1 / math.sqrt(ms + 1e-5)) * w[i], rel=1e-12)


def test_rotary_full_head_is_the_reference_loop():
    rng = np.random.default_rng(1)
    heads, hd, theta = 3, 8, 10000.0
    x = rng.normal(size=(5, heads * hd))
    pos = np.arange(5) + 7
    out = pm.rotary(x, heads, hd, hd, theta, pos)
    half = hd // 2
    for i in range(5):
        for h in range(heads):
            for j in range(half):                                # src/minimax.rs:75-81
                ang = float(pos[i]) * (1.0 / theta ** (2.0 * j / hd))
                a, b = x[i, h * hd + j], x[i, h * hd + j + half]
                assert out[i, h * hd + j] == pytest.approx(a * math.cos(ang) - b * math.sin(ang), rel=1e-9, abs=1e-12)
                assert out[i, h * hd + j + half] == pytest.approx(b * math.cos(ang) + a * math.sin(ang), rel=1e-9, abs=1e-12)


def test_partial_rotary_leaves_the_rest():
    rng = np.random.default_rng(2)
    x = rng.normal(size=(4, 2 * 12))
    out = pm.rotary(x, 2, 12, 6, 500.0, np.arange(4))
    for h in range(2):
        np.testing.assert_array_equal(out[:, h * 12 + 6:(h + 1) * 12], x[:, h * 12 + 6:(h + 1) * 12])
    assert not np.allclose(out[1:, :6], x[1:, :6])
    np.testing.assert_allclose(out[0], x[0])                    # position 0 rotates by nothing
    norms = lambda v: np.linalg.norm(v.reshape(4, 2, 12)[:, :, :6], axis=-1)
    np.testing.assert_allclose(norms(out), norms(x))


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(3)
    T, nh, nkv, hd = 9, 4, 2, 6
    q, k, v = rng.normal(size=(T, nh * hd)), rng.normal(size=(T, nkv * hd)), rng.normal(size=(T, nkv * hd))
    out = pm.causal_attention(q, k, v, nh, nkv, hd, hd ** -0.5)
    np.testing.assert_allclose(out[:5], pm.causal_attention(q[:5], k[:5], v[:5], nh, nkv, hd, hd ** -0.5))
    for h in range(nh):                                          # row 0 sees key 0 only
        np.testing.assert_allclose(out[0, h * hd:(h + 1) * hd], v[0, (h // 2) * hd:(h // 2 + 1) * hd])
    k2 = k.copy(); k2[:, :hd] += rng.normal(size=(T, hd))                            # kv head 0 feeds query heads 0 and 1 only
    out2 = pm.causal_attention(q, k2, v, nh, nkv, hd, hd ** -0.5)
    assert not np.allclose(out2[:, :2 * hd], out[:, :2 * hd]) and np.allclose(out2[:, 2 * hd:], out[:, 2 * hd:])
    win = pm.causal_attention(q, k, v, nh, nkv, hd, hd ** -0.5, window=3)
    np.testing.assert_allclose(win[:3], out[:3])
    np.testing.assert_allclose(win[8], pm.causal_attention(q[6:], k[6:], v[6:], nh, nkv, hd, hd ** -0.5)[2])


def test_attention_of_chosen_rows_is_the_rows_of_the_whole():
    rng = np.random.default_rng(31)
    T, nh, nkv, hd = 40, 4, 2, 6
    q, k, v = rng.normal(size=(T, nh * hd)), rng.normal(size=(T, nkv * hd)), rng.normal(size=(T, nkv * hd))
    rows = [0, 17, 39]
    for window in (None, 9):
        whole = pm.causal_attention(q, k, v, nh, nkv, hd, 0.3, window=window)
        np.testing.assert_allclose(pm.causal_attention(q[rows], k, v, nh, nkv, hd, 0.3, window=window, rows=rows), whole[rows])


def test_router_bias_decides_choice_only_ties_go_low_and_weights_sum_to_one():
    rng = np.random.default_rng(4)
    a2, W = rng.normal(size=(6, 10)), rng.normal(size=(5, 10))
    ids0, w0, _ = pm.route(a2, W, np.zeros(5), 2)
    np.testing.assert_allclose(w0.sum(-1), 1.0)
    bias = np.array([0, 0, 0, 0, 10.0])
    ids1, w1, _ = pm.route(a2, W, bias, 2)
    assert (ids1[:, 0] == 4).all()
    score = 1 / (1 + np.exp(-(a2 @ W.T)))
    for t in range(6):
        picked = score[t, ids1[t]]
        np.testing.assert_allclose(w1[t], picked / picked.sum())         # the bias is not in the weights
    ids2, _, margin = pm.route(np.zeros((1, 10)), W, np.zeros(5), 3)       # all scores 0.5: ties
    assert ids2.tolist() == [[0, 1, 2]] and margin[0] == 0.0


def test_experts_are_summed_with_their_weights():
    config, init = ALL["b"]
    s = pm.sizes_from_config(config)
    rng = np.random.default_rng(5)
    W = {"model.layers.0.block_sparse_moe.gate.weight": rng.normal(size=(8, 96)),
         "model.layers.0.block_sparse_moe.e_score_correction_bias": rng.normal(size=8) * 0.1}
    for e in range(8):
        W[f"model.layers.0.block_sparse_moe.experts.{e}.w1.weight"] = rng.normal(size=(48, 96)) * 0.1
        W[f"model.layers.0.block_sparse_moe.experts.{e}.w3.weight"] = rng.normal(size=(48, 96)) * 0.1
        W[f"model.layers.0.block_sparse_moe.experts.{e}.w2.weight"] = rng.normal(size=(96, 48)) * 0.1
    a2 = rng.normal(size=(4, 96))
    out, _ = pm.routed_experts(a2, W, "model.layers.0.", s)
    ids, w, _ = pm.route(a2, W["model.layers.0.block_sparse_moe.gate.weight"],
                         W["model.layers.0.block_sparse_moe.e_score_correction_bias"], 3)
    t = 2
    want = np.zeros(96)
    for r in range(3):
        e = ids[t, r]
        g = a2[t] @ W[f"model.layers.0.block_sparse_moe.experts.{e}.w1.weight"].T
        u = a2[t] @ W[f"model.layers.0.block_sparse_moe.experts.{e}.w3.weight"].T
        want += w[t, r] * ((g / (1 + np.exp(-g)) * u) @ W[f"model.layers.0.block_sparse_moe.experts.{e}.w2.weight"].T)
    np.testing.assert_allclose(out[t], want, rtol=1e-10)


@pytest.mark.parametrize("name", list(ALL))
def test_whole_model_prefix_property_and_precisions(tmp_path, name):
    config, init = ALL[name]
    folder = str(tmp_path / name)
    fr.write_random_model(folder, config, init)
    cfg, W = pm.read_model_folder(folder)
    ids = np.random.default_rng(6).integers(0, cfg["vocab_size"], size=20).tolist()
    full = pm.logits_all_positions(cfg, W, ids)
    assert full.shape == (20, cfg["vocab_size"]) and np.isfinite(full).all()
    np.testing.assert_allclose(pm.logits_all_positions(cfg, W, ids[:11]), full[:11], rtol=1e-9, atol=1e-12)
    single = pm.logits_all_positions(cfg, W, ids, dtype=np.float32)
    assert np.abs(single - full).max() < 2e-4 * max(1.0, np.abs(full).max())
    assert np.std(full) > 1e-3                                    # the weights do something


def test_greedy_generation_and_stop_rule(tmp_path):
    config, init = ALL["a"]
    folder = str(tmp_path / "a")
    fr.write_random_model(folder, config, init)
    cfg, W = pm.read_model_folder(folder)
    out = pm.generate_greedy(cfg, W, [3, 4, 5], 6)
    assert len(out) == 6
    assert out[0] == pm.greedy_pick(pm.logits_all_positions(cfg, W, [3, 4, 5])[-1])
    assert pm.generate_greedy(cfg, W, [3, 4, 5], 6, eos=(out[2],)) == out[:2]
    assert pm.greedy_pick([1.0, 3.0, 3.0, 2.0]) == 2              # the last of equal maxima
    assert pm.temperature_pick([0.0, 0.0, 0.0, 0.0], 1.0, 0.6) == 2


def test_sampling_floor_and_pick_among_the_kept():
    row = np.log(np.array([0.05, 0.4, 0.1, 0.25, 0.2]))
    assert pm.sampling_floor(row, 1.0) == -np.inf
    assert pm.sampling_floor(row, 1.0, top_k=2) == row[3]
    assert pm.sampling_floor(row, 1.0, top_p=0.6) == row[3]          # 0.4 + 0.25 reaches 0.6
    assert pm.sampling_floor(row, 1.0, top_p=0.66) == row[4]         # 0.65 does not reach 0.66: 0.2 stays too
    assert pm.sampling_floor(row, 1.0, top_k=1, top_p=0.9) == row[1]
    # among the kept {1, 3}: probabilities 0.4 / 0.65 and 0.25 / 0.65, in index order
    assert pm.top_k_top_p_pick(row, 1.0, 0.5, top_k=2) == 1
    assert pm.top_k_top_p_pick(row, 1.0, 0.7, top_k=2) == 3
    assert pm.top_k_top_p_pick(row, 1.0, 0.999, top_p=0.6) == 3

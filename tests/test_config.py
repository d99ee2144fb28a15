import json
import os

import pytest

import fieldrun_b200 as fr
from fieldrun_b200.config import ConfigError, architecture_for, load_config
from tiny_configs import CONFIG_A, CONFIG_B, CONFIG_C


def test_reads_every_key():
    cfg = fr.MiniMaxM2Config.from_dict(CONFIG_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 6, 2)
    assert (cfg.head_dim, cfg.rotary_dim, cfg.rope_theta, cfg.use_qk_norm) == (32, 32, 1e6, False)
    assert (cfg.num_local_experts, cfg.num_experts_per_tok, cfg.intermediate_size) == (8, 3, 48)
    assert (cfg.vocab_size, cfg.rms_norm_eps, cfg.eos_token_id) == (389, 1e-5, (7, 11))


def test_defaults_follow_the_reference():
    raw = dict(architectures=["MiniMaxM2ForCausalLM"], num_hidden_layers=1, hidden_size=48, num_attention_heads=4,
               num_experts=3, num_experts_per_tok=2, intermediate_size=8, vocab_size=10)
    cfg = fr.MiniMaxM2Config.from_dict(raw)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 12 and cfg.rotary_dim == 12
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6 and cfg.use_qk_norm and not cfg.tie_word_embeddings
    assert cfg.eos_token_id == ()
    raw["rope_parameters"] = {"rope_theta": 777.0}
    assert fr.MiniMaxM2Config.from_dict(raw).rope_theta == 777.0


def test_partial_rotary_factor_and_experts_alias():
    cfg = fr.MiniMaxM2Config.from_dict(CONFIG_C)
    assert cfg.rotary_dim == 6 and cfg.num_local_experts == 5 and cfg.tie_word_embeddings


@pytest.mark.parametrize("key", ["hidden_size", "num_attention_heads", "num_hidden_layers", "vocab_size",
                                 "intermediate_size", "num_experts_per_tok"])
def test_missing_key_is_named(key):
    raw = dict(CONFIG_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        fr.MiniMaxM2Config.from_dict(raw)


@pytest.mark.parametrize("change, word", [
    (dict(num_key_value_heads=3), "num_key_value_heads"), (dict(rotary_dim=7), "rotary_dim"),
    (dict(rotary_dim=18), "rotary_dim"), (dict(num_experts_per_tok=9), "num_experts_per_tok"),
    (dict(hidden_size="64"), "hidden_size"),
    (dict(scoring_func="softmax"), "scoring_func"), (dict(rms_norm_eps=0), "rms_norm_eps"),
])
def test_bad_values_are_named(change, word):
    with pytest.raises(ConfigError, match=word):
        fr.MiniMaxM2Config.from_dict({**CONFIG_A, **change})


FIXTURES = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures")


def test_a_config_in_the_form_the_architectures_writer_emits(capsys):
    """tests/fixtures/written_config_tiny.json has the keys and nesting that the architecture's own writer
    produces for the tiny model of the reference's gate (scripts/gemma3_ref.py:61-77): theta and the rotary
    share under ``rope_parameters``, the family's default stop token 200020 although the vocabulary is 64,
    and bookkeeping keys the model has no use for."""
    with open(os.path.join(FIXTURES, "written_config_tiny.json")) as handle:
        raw = json.load(handle)
    cfg = fr.MiniMaxM2Config.from_dict(raw)
    assert "200020" in capsys.readouterr().err            # said once, then dropped
    assert cfg.eos_token_id == ()
    assert (cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers) == (64, 32, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (4, 2, 8)
    assert cfg.rotary_dim == 4 and cfg.rope_theta == 5e6 and cfg.rms_norm_eps == 1e-6
    assert (cfg.num_local_experts, cfg.num_experts_per_tok, cfg.intermediate_size) == (8, 2, 16)
    assert cfg.use_qk_norm and cfg.use_routing_bias and not cfg.tie_word_embeddings
    # the plain implementation reads the same file on its own
    import plain_model as pm
    s = pm.sizes_from_config(raw)
    assert (s["rotary"], s["theta"], s["hd"], s["nkv"], s["experts"], s["top_k"]) == (4, 5e6, 8, 2, 8, 2)


def test_a_config_with_the_published_checkpoints_keys():
    """The full-size form: ``rotary_dim`` and ``rope_theta`` at the top level, null stop tokens, and the
    family's keys that this architecture fixes (all layers softmax attention, no shared expert, betas of 1)."""
    with open(os.path.join(FIXTURES, "written_config_full_size.json")) as handle:
        cfg = fr.MiniMaxM2Config.from_dict(json.load(handle))
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (3072, 48, 8, 128)
    assert (cfg.rotary_dim, cfg.rope_theta, cfg.rms_norm_eps) == (64, 5e6, 1e-6)
    assert (cfg.num_local_experts, cfg.num_experts_per_tok, cfg.intermediate_size) == (256, 8, 1536)
    assert (cfg.vocab_size, cfg.num_hidden_layers, cfg.eos_token_id) == (200064, 62, ())


def test_the_rotary_share_in_each_of_its_spellings():
    base = {k: v for k, v in CONFIG_A.items() if k not in ("rotary_dim", "rope_theta")}            # head_dim 16
    assert fr.MiniMaxM2Config.from_dict(base).rotary_dim == 16
    assert fr.MiniMaxM2Config.from_dict({**base, "rotary_dim": 8}).rotary_dim == 8
    assert fr.MiniMaxM2Config.from_dict({**base, "partial_rotary_factor": 0.5}).rotary_dim == 8
    nested = {**base, "rope_parameters": {"partial_rotary_factor": 0.5, "rope_theta": 123.0, "rope_type": "default"}}
    cfg = fr.MiniMaxM2Config.from_dict(nested)
    assert cfg.rotary_dim == 8 and cfg.rope_theta == 123.0
    assert fr.MiniMaxM2Config.from_dict({**nested, "rotary_dim": 8}).rotary_dim == 8      # agreeing twice is fine
    with pytest.raises(ConfigError, match="rotary share"):
        fr.MiniMaxM2Config.from_dict({**nested, "rotary_dim": 16})
    with pytest.raises(ConfigError, match="rotary share"):
        fr.MiniMaxM2Config.from_dict({**nested, "partial_rotary_factor": 0.25})


def test_stop_tokens_outside_the_vocabulary_are_dropped_not_refused(capsys):
    cfg = fr.MiniMaxM2Config.from_dict({**CONFIG_A, "eos_token_id": [3, 999, 255, -1]})
    assert cfg.eos_token_id == (3, 255)
    err = capsys.readouterr().err
    assert "999" in err and "-1" in err and err.count("\n") == 1


@pytest.mark.parametrize("change, word", [
    (dict(sliding_window=128), "sliding_window"),
    (dict(rope_parameters={"rope_type": "yarn", "factor": 4.0}), "rope_type"),
    (dict(rope_scaling={"type": "linear", "factor": 2.0}), "rope_scaling"),
    (dict(shared_intermediate_size=64), "shared_intermediate_size"),
    (dict(n_shared_experts=1), "n_shared_experts"),
    (dict(norm_topk_prob=False), "norm_topk_prob"),
    (dict(routed_scaling_factor=2.5), "routed_scaling_factor"),
    (dict(scoring_func="softmax"), "scoring_func"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(attn_type_list=[1, 0]), "attn_type_list"),
    (dict(layer_types=["full_attention", "sliding_attention"]), "layer_types"),
    (dict(qk_norm_type="per_head"), "qk_norm_type"),
    (dict(layernorm_mlp_beta=0.5), "layernorm_mlp_beta"),
    (dict(n_group=4), "n_group"),
    (dict(final_logit_softcapping=30.0), "final_logit_softcapping"),
])
def test_keys_that_would_change_the_arithmetic_are_refused_by_name(change, word):
    with pytest.raises(ConfigError, match=word):
        fr.MiniMaxM2Config.from_dict({**CONFIG_A, **change})


def test_the_same_keys_with_harmless_values_pass():
    harmless = dict(sliding_window=None, rope_parameters={"rope_type": "default", "rope_theta": 10000.0},
                    rope_scaling=None, shared_intermediate_size=0, norm_topk_prob=True, routed_scaling_factor=1.0,
                    hidden_act="silu", attention_bias=False, attn_type_list=[1, 1], layernorm_mlp_beta=1.0,
                    qk_norm_type="per_layer", n_group=1, final_logit_softcapping=None)
    cfg = fr.MiniMaxM2Config.from_dict({**{k: v for k, v in CONFIG_A.items() if k != "rope_theta"}, **harmless})
    assert cfg == fr.MiniMaxM2Config.from_dict(CONFIG_A)


def test_a_model_without_a_routing_bias():
    cfg = fr.MiniMaxM2Config.from_dict({**CONFIG_A, "use_routing_bias": False})
    arch = architecture_for(CONFIG_A)
    ff = arch.plan(cfg).layers[0].feed_forward
    assert ff.args["choice_bias"] is False
    names = [n.name for n in fr.build_model(arch, cfg, "float32").tensor_needs()]
    assert not any("e_score_correction_bias" in n for n in names)


def test_registry_by_architecture_and_model_type():
    assert architecture_for(CONFIG_A).name == "MiniMaxM2ForCausalLM"
    assert architecture_for({"model_type": "minimax_m2"}).name == "MiniMaxM2ForCausalLM"
    with pytest.raises(ConfigError, match="registered: MiniMaxM2ForCausalLM"):
        architecture_for({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_config_json_round_trip(tmp_path):
    for raw in (CONFIG_A, CONFIG_B, CONFIG_C):
        cfg = fr.MiniMaxM2Config.from_dict(raw)
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_json_dict()))
        arch, again = load_config(str(tmp_path))
        assert again == cfg and arch.name == cfg.architecture


def test_plan_is_data():
    arch = architecture_for(CONFIG_B)
    plan = arch.plan(arch.config_from_dict(CONFIG_B, "c"))
    assert len(plan.layers) == 3 and [r.layer for r in plan.run_order] == [0, 1, 2]
    mixer = plan.layers[1].mixer
    assert mixer.kind == "gqa_attention" and mixer.args["qk_norm"] == "none" and mixer.args["window"] is None
    assert mixer.args["position"]["rotary_dim"] == 32 and "q_norm" not in mixer.tensors
    ff = plan.layers[2].feed_forward
    assert ff.kind == "routed_experts" and ff.args["top_k"] == 3 and ff.args["choice_bias"]
    assert ff.tensors["w_down"] == "model.layers.2.block_sparse_moe.experts.{e}.w2.weight"


def test_rotary_tables_are_the_reference_angles():
    """cos/sin of pos * theta^(-2j/rotary_dim) (src/minimax.rs:50,76), to float32 rounding."""
    import numpy as np
    from fieldrun_b200.parts.position import Rotary
    cos, sin = Rotary({"rotary_dim": 12, "theta": 5000000.0}).tables(300, "cpu")
    assert cos.shape == (300, 6) and cos.dtype.is_floating_point
    pos, j = np.arange(300)[:, None], np.arange(6)[None, :]
    angle = pos * (1.0 / 5000000.0 ** (2.0 * j / 12))
    np.testing.assert_allclose(cos.numpy(), np.cos(angle), atol=1e-7)
    np.testing.assert_allclose(sin.numpy(), np.sin(angle), atol=1e-7)
    scaled, _ = Rotary({"rotary_dim": 12, "theta": 5000000.0, "position_scale": 0.5}).tables(300, "cpu")
    np.testing.assert_allclose(scaled.numpy()[2 * np.arange(100)], cos.numpy()[:100], atol=1e-7)
    assert Rotary({"rotary_dim": 0, "theta": 1.0}).tables(10, "cpu") == (None, None)
    with pytest.raises(ValueError, match="even"):
        Rotary({"rotary_dim": 5, "theta": 1.0})


def test_rotary_tables_far_out_and_the_references_float32_recipe():
    """The reference forms the angle in float32: inv[j] = 1 / theta.powf(2j / R) (src/minimax.rs:50) and
    ang = (pos as f32) * inv[j] (src/minimax.rs:76).  At position 65,535 a float32 angle of the fastest pair is
    only known to half a unit in its last place (2^-9 rad = 2.0e-3) plus the position times the rounding of inv
    (65,535 x 3e-8 = 2.0e-3): two float32 routines (another powf, a fused multiply) differ by that much among
    themselves.  The library's tables are computed in float64 and rounded once, which lies inside that band;
    this test states the band and that the tables are within it, from the first position to the 65,536th."""
    import numpy as np
    from fieldrun_b200.parts.position import Rotary
    theta, rotary_dim = 5000000.0, 64
    cos, sin = Rotary({"rotary_dim": rotary_dim, "theta": theta}).tables(65536, "cpu")
    j = np.arange(rotary_dim // 2, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(theta), np.float32(2.0) * j / np.float32(rotary_dim))).astype(np.float32)
    for first, end, band in ((0, 300, 3e-5), (60000, 65536, 6e-3)):
        pos = np.arange(first, end).astype(np.float32)
        ang = (pos[:, None] * inv[None, :]).astype(np.float32)               # the product rounded to float32
        for table, fn in ((cos, np.cos), (sin, np.sin)):
            diff = np.abs(table[first:end].numpy().astype(np.float64) - fn(ang.astype(np.float64)))
            assert diff.max() < band, (first, diff.max())
            if first:
                assert diff.max() > 1e-4                                  # far out the two recipes do part: by the band, not more
                assert diff[:, 16:].max() < 2e-5                          # and only in the fast pairs; the slow ones agree
    exact = np.arange(60000, 65536, dtype=np.float64)[:, None] * (1.0 / theta ** (2.0 * np.arange(32) / rotary_dim))[None, :]
    assert np.abs(cos[60000:].numpy() - np.cos(exact)).max() < 1e-7       # the tables are the exact angles, rounded once

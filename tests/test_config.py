import json

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
    (dict(eos_token_id=999), "eos_token_id"), (dict(hidden_size="64"), "hidden_size"),
    (dict(scoring_func="softmax"), "scoring_func"), (dict(rms_norm_eps=0), "rms_norm_eps"),
])
def test_bad_values_are_named(change, word):
    with pytest.raises(ConfigError, match=word):
        fr.MiniMaxM2Config.from_dict({**CONFIG_A, **change})


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

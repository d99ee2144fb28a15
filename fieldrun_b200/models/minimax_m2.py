"""MiniMax-M2 as a plan of parts.

Every layer is: RMSNorm -> grouped-query attention with one RMSNorm over the
whole Q projection and one over the whole K projection, then rotary on the first
``rotary_dim`` dims of each head -> residual; RMSNorm -> experts routed by a
sigmoid score whose correction bias only decides the choice -> residual
(src/minimax.rs:128-160 for whole prompts, :253-287 with a cache).  Tensor names
are the checkpoint's own (src/convert.rs:1231-1257): ``block_sparse_moe.gate``,
``e_score_correction_bias`` and per expert ``w1`` (gate), ``w3`` (up), ``w2`` (down).
"""
from __future__ import annotations

from ..config.minimax_m2 import ARCHITECTURE, MiniMaxM2Config
from ..config.plan import LayerSpec, ModelPlan, PartSpec, default_run_order
from ..config.registry import Architecture, register_architecture


def minimax_m2_plan(cfg: MiniMaxM2Config) -> ModelPlan:
    d = cfg.hidden_size
    layers = []
    for index in range(cfg.num_hidden_layers):
        p = f"model.layers.{index}."
        moe = p + "block_sparse_moe."
        attention_tensors = {
            "q_proj": p + "self_attn.q_proj.weight",
            "k_proj": p + "self_attn.k_proj.weight",
            "v_proj": p + "self_attn.v_proj.weight",
            "o_proj": p + "self_attn.o_proj.weight",
        }
        if cfg.use_qk_norm:
            attention_tensors["q_norm"] = p + "self_attn.q_norm.weight"
            attention_tensors["k_norm"] = p + "self_attn.k_norm.weight"
        mixer = PartSpec(
            kind="gqa_attention",
            args={
                "hidden_size": d,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                # one RMS over the whole projection row, before the head split (src/minimax.rs:137-138)
                "qk_norm": "full_width" if cfg.use_qk_norm else "none",
                "qk_norm_eps": cfg.rms_norm_eps,
                "position": {"kind": "rotary", "rotary_dim": cfg.rotary_dim, "theta": cfg.rope_theta,
                             "pairing": "half"},
                "softmax_scale": float(cfg.head_dim) ** -0.5,   # src/minimax.rs:51
                "window": None,                                  # full attention in every layer
            },
            tensors=attention_tensors,
        )
        feed_forward = PartSpec(
            kind="routed_experts",
            args={
                "hidden_size": d,
                "num_experts": cfg.num_local_experts,
                "top_k": cfg.num_experts_per_tok,
                "expert_width": cfg.intermediate_size,
                "score": "sigmoid",            # src/minimax.rs:95
                "choice_bias": cfg.use_routing_bias,   # the bias enters the choice only, src/minimax.rs:96-101
                "renormalize": True,           # weights are sig / sum of picked sig, src/minimax.rs:100-103
                "routed_scale": 1.0,
            },
            tensors={
                "router": moe + "gate.weight",
                "choice_bias": moe + "e_score_correction_bias",
                "w_gate": moe + "experts.{e}.w1.weight",
                "w_up": moe + "experts.{e}.w3.weight",
                "w_down": moe + "experts.{e}.w2.weight",
            },
        )
        layers.append(LayerSpec(
            block="pre_norm",
            mixer=mixer,
            feed_forward=feed_forward,
            mixer_norm=PartSpec("rmsnorm", {"width": d, "eps": cfg.rms_norm_eps},
                                {"weight": p + "input_layernorm.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {"width": d, "eps": cfg.rms_norm_eps},
                                       {"weight": p + "post_attention_layernorm.weight"}),
        ))
    embedding_name = "model.embed_tokens.weight"
    plan = ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=d,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": d},
                           {"weight": embedding_name}),
        layers=tuple(layers),
        run_order=default_run_order(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {"width": d, "eps": cfg.rms_norm_eps}, {"weight": "model.norm.weight"}),
        # untied unless tie_word_embeddings, then the embedding rows (src/minimax.rs:54, src/convert.rs:1234-1236)
        head=PartSpec("vocab_head", {"vocab_size": cfg.vocab_size, "width": d},
                      {"weight": embedding_name if cfg.tie_word_embeddings else "lm_head.weight"}),
        eos_token_id=cfg.eos_token_id,
    )
    plan.check()
    return plan


register_architecture(Architecture(
    name=ARCHITECTURE,
    config_from_dict=MiniMaxM2Config.from_dict,
    plan=minimax_m2_plan,
    model_type_prefixes=("minimax",),
), replace=True)

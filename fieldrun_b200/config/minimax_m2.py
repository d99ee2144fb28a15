"""Configuration of the MiniMax-M2 architecture, read from its own config.json keys.

Keys and defaults follow the reference's converter for this architecture
(src/convert.rs:1208-1219 and rope_theta_eps at src/convert.rs:610-615):
``num_key_value_heads`` defaults to ``num_attention_heads``, ``head_dim`` to
``hidden_size / num_attention_heads``, ``rope_theta`` (or
``rope_parameters.rope_theta``) to 10000, ``rms_norm_eps`` to 1e-6,
``tie_word_embeddings`` to false; experts are counted by ``num_local_experts``
or ``num_experts``; ``eos_token_id`` is an int or a list (src/convert.rs:375-381).

Three keys go beyond what the reference reads: ``rotary_dim`` (or
``partial_rotary_factor``, at the top level or under ``rope_parameters``), the
number of leading dims of each head that are rotated (the reference rotates the
whole head, src/minimax.rs:50,69-84, and has the partial form in
src/qwen35moe.rs:78-81,121-138); ``use_qk_norm`` (the reference always norms,
src/minimax.rs:137-138); ``use_routing_bias`` (false: no choice bias tensor).
Keys of this family of checkpoints that would change the arithmetic and are not
built (a window, scaled rotary angles, a shared expert, unnormalised or scaled
routing weights, biases, capped logits) are refused by name, never ignored.
"""
from __future__ import annotations

import sys
from dataclasses import asdict, dataclass
from typing import Any, Mapping

from .base import ConfigError, KeyReader, ModelConfig

ARCHITECTURE = "MiniMaxM2ForCausalLM"


def _rotary_dim(r: KeyReader, head_dim: int, where: str) -> int:
    """How many leading dims of each head are rotated.  Three spellings exist: ``rotary_dim`` (a count),
    ``partial_rotary_factor`` at the top level and ``rope_parameters.partial_rotary_factor`` (shares of the
    head, ``int(head_dim * factor)`` as src/convert.rs:965-966 computes it for its partial-rotary
    architecture; ``rope_parameters`` is where the reference also looks for theta, src/convert.rs:610-615).
    Whichever are present must agree; with none the whole head is rotated (src/minimax.rs:50,69-84)."""
    found: dict[str, int] = {}
    if r.present("rotary_dim"):
        found["rotary_dim"] = r.integer("rotary_dim", minimum=0)
    for name in ("partial_rotary_factor", "rope_parameters.partial_rotary_factor"):
        if r.present(name):
            found[name] = int(head_dim * r.real(name, positive=True))
    if len(set(found.values())) > 1:
        raise ConfigError(f"{where}: the rotary share is given more than once and differently: "
                          + ", ".join(f"{k!r} -> {v} dims" for k, v in found.items()))
    return next(iter(found.values()), head_dim)


def _stop_tokens(ids: tuple[int, ...], vocab: int, where: str) -> tuple[int, ...]:
    """The reference reads ``eos_token_id`` without a range check (src/convert.rs:375-381): an id outside the
    vocabulary can never be produced, so it stops nothing.  Such ids are dropped, with one line on stderr."""
    kept = tuple(t for t in ids if 0 <= t < vocab)
    if len(kept) != len(ids):
        dropped = [t for t in ids if not 0 <= t < vocab]
        print(f"{where}: eos_token_id {dropped} lies outside the vocabulary of {vocab} and can never be "
              f"produced; ignored", file=sys.stderr)
    return kept


def _one(value) -> bool:
    return float(value) == 1.0


# key -> (what its value must satisfy, why anything else is refused).  These keys belong to this family of
# checkpoints (or to its writers) and change the arithmetic; the reference reads none of them
# (src/convert.rs:1208-1219) and its forward has one fixed form (src/minimax.rs:88-160).
_NOT_BUILT = (
    ("scoring_func", lambda v: v == "sigmoid", "this architecture routes with 'sigmoid' scores (src/minimax.rs:95)"),
    ("hidden_act", lambda v: v in ("silu", "swish"), "the experts are gated with silu (src/minimax.rs:31,116-119)"),
    ("sliding_window", lambda v: int(v) <= 0, "every layer attends to all earlier keys (src/minimax.rs:270-281); "
                                              "a window is not part of this architecture"),
    ("rope_parameters.rope_type", lambda v: v == "default", "only unscaled rotary angles are built (src/minimax.rs:50,76)"),
    ("rope_parameters.type", lambda v: v == "default", "only unscaled rotary angles are built (src/minimax.rs:50,76)"),
    ("rope_scaling", lambda v: isinstance(v, Mapping) and v.get("rope_type", v.get("type", "default")) == "default",
     "only unscaled rotary angles are built (src/minimax.rs:50,76)"),
    ("shared_intermediate_size", lambda v: int(v) == 0, "a shared expert is not part of this architecture (src/minimax.rs:88-126)"),
    ("n_shared_experts", lambda v: int(v) == 0, "a shared expert is not part of this architecture (src/minimax.rs:88-126)"),
    ("num_shared_experts", lambda v: int(v) == 0, "a shared expert is not part of this architecture (src/minimax.rs:88-126)"),
    ("norm_topk_prob", lambda v: v is True, "the picked weights are always renormalised (src/minimax.rs:100-103)"),
    ("routed_scaling_factor", _one, "the experts' sum is not scaled (src/minimax.rs:121-123)"),
    ("n_group", lambda v: int(v) <= 1, "experts are chosen among all of them, not by groups (src/minimax.rs:96-99)"),
    ("topk_group", lambda v: int(v) <= 1, "experts are chosen among all of them, not by groups (src/minimax.rs:96-99)"),
    ("attention_bias", lambda v: v is False, "the projections have no bias (src/minimax.rs:262-264)"),
    ("qkv_bias", lambda v: v is False, "the projections have no bias (src/minimax.rs:262-264)"),
    ("mlp_bias", lambda v: v is False, "the experts have no bias (src/minimax.rs:116-120)"),
    ("attn_type_list", lambda v: all(int(t) == 1 for t in v), "every layer is softmax attention (src/minimax.rs:253-282)"),
    ("layer_types", lambda v: all(t == "full_attention" for t in v), "every layer is full attention (src/minimax.rs:253-282)"),
    ("qk_norm_type", lambda v: v == "per_layer", "q and k are normed over the whole projection row (src/minimax.rs:137-138)"),
    ("layernorm_full_attention_beta", _one, "the residual stream is not scaled (src/minimax.rs:282-284)"),
    ("layernorm_linear_attention_beta", _one, "the residual stream is not scaled (src/minimax.rs:282-284)"),
    ("layernorm_mlp_beta", _one, "the residual stream is not scaled (src/minimax.rs:282-284)"),
    ("attn_logit_softcapping", lambda v: False, "scores are not capped (src/minimax.rs:270-281)"),
    ("final_logit_softcapping", lambda v: False, "logits are not capped (src/minimax.rs:373-376)"),
    ("mlp_only_layers", lambda v: len(v) == 0, "every layer's feed-forward is routed experts (src/minimax.rs:88-126)"),
    ("first_k_dense_replace", lambda v: int(v) == 0, "every layer's feed-forward is routed experts (src/minimax.rs:88-126)"),
)


def _refuse_what_is_not_built(r: KeyReader) -> None:
    for name, allowed, why in _NOT_BUILT:
        r.refuse_unless(name, allowed, why)


@dataclass(frozen=True)
class MiniMaxM2Config(ModelConfig):
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rotary_dim: int = 0
    rope_theta: float = 10000.0
    use_qk_norm: bool = True
    rms_norm_eps: float = 1e-6
    num_local_experts: int = 0
    num_experts_per_tok: int = 0
    intermediate_size: int = 0
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 0
    use_routing_bias: bool = True

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "MiniMaxM2Config":
        r = KeyReader(raw, where)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        if not r.present("head_dim"):
            if hidden % heads:
                raise ConfigError(
                    f"{where}: 'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}")
            head_dim = hidden // heads
        else:
            head_dim = r.integer("head_dim", minimum=2)
        rotary = _rotary_dim(r, head_dim, where)
        _refuse_what_is_not_built(r)
        vocab = r.integer("vocab_size", minimum=1)
        cfg = cls(
            architecture=ARCHITECTURE,
            vocab_size=vocab,
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            eos_token_id=_stop_tokens(r.integer_list("eos_token_id", default=()), vocab, where),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rotary_dim=rotary,
            rope_theta=r.real("rope_theta", "rope_parameters.rope_theta", default=10000.0, positive=True),
            use_qk_norm=r.boolean("use_qk_norm", default=True),
            rms_norm_eps=r.real("rms_norm_eps", default=1e-6, positive=True),
            num_local_experts=r.integer("num_local_experts", "num_experts", minimum=1),
            num_experts_per_tok=r.integer("num_experts_per_tok", minimum=1),
            intermediate_size=r.integer("intermediate_size", minimum=1),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            max_position_embeddings=r.integer("max_position_embeddings", default=0, minimum=0),
            use_routing_bias=r.boolean("use_routing_bias", default=True),
        )
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"{where}: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"{where}: head_dim {self.head_dim} must be even")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ConfigError(
                f"{where}: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        if self.num_experts_per_tok > self.num_local_experts:
            raise ConfigError(
                f"{where}: num_experts_per_tok {self.num_experts_per_tok} exceeds "
                f"num_local_experts {self.num_local_experts}")
        for token in self.eos_token_id:
            if not 0 <= token < self.vocab_size:
                raise ConfigError(f"{where}: stop token {token} is outside the vocabulary of {self.vocab_size}")

    def to_json_dict(self) -> dict[str, Any]:
        """The config.json that reads back to this configuration."""
        out = asdict(self)
        out.pop("architecture")
        out["architectures"] = [ARCHITECTURE]
        out["model_type"] = "minimax_m2"
        eos = out.pop("eos_token_id")
        if len(eos) == 1:
            out["eos_token_id"] = eos[0]
        elif eos:
            out["eos_token_id"] = list(eos)
        out["scoring_func"] = "sigmoid"
        if not out["max_position_embeddings"]:
            out.pop("max_position_embeddings")
        return out

"""Configuration of the MiniMax-M2 architecture, read from its own config.json keys.

Keys and defaults follow the reference's converter for this architecture
(src/convert.rs:1208-1219 and rope_theta_eps at src/convert.rs:610-615):
``num_key_value_heads`` defaults to ``num_attention_heads``, ``head_dim`` to
``hidden_size / num_attention_heads``, ``rope_theta`` (or
``rope_parameters.rope_theta``) to 10000, ``rms_norm_eps`` to 1e-6,
``tie_word_embeddings`` to false; experts are counted by ``num_local_experts``
or ``num_experts``; ``eos_token_id`` is an int or a list (src/convert.rs:375-381).

Two keys go beyond what the reference reads: ``rotary_dim`` (or
``partial_rotary_factor``), the number of leading dims of each head that are
rotated (the reference rotates the whole head, src/minimax.rs:50,69-84, and has
the partial form in src/qwen35moe.rs:78-81,121-138), and ``use_qk_norm`` (the
reference always norms, src/minimax.rs:137-138).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping

from .base import ConfigError, KeyReader, ModelConfig

ARCHITECTURE = "MiniMaxM2ForCausalLM"


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

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "MiniMaxM2Config":
        r = KeyReader(raw, where)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        if "head_dim" not in raw or raw["head_dim"] is None:
            if hidden % heads:
                raise ConfigError(
                    f"{where}: 'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}")
            head_dim = hidden // heads
        else:
            head_dim = r.integer("head_dim", minimum=2)
        if "rotary_dim" in raw and raw["rotary_dim"] is not None:
            rotary = r.integer("rotary_dim", minimum=0)
        elif "partial_rotary_factor" in raw and raw["partial_rotary_factor"] is not None:
            # int(head_dim * factor), as the reference does for its partial-rotary arch (src/convert.rs:965-966)
            rotary = int(head_dim * r.real("partial_rotary_factor", positive=True))
        else:
            rotary = head_dim
        scoring = r.text("scoring_func", default="sigmoid")
        if scoring != "sigmoid":
            raise ConfigError(f"{where}: key 'scoring_func' is {scoring!r}; this architecture routes with 'sigmoid'")
        cfg = cls(
            architecture=ARCHITECTURE,
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            eos_token_id=r.integer_list("eos_token_id", default=()),
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
                raise ConfigError(f"{where}: eos_token_id {token} is outside the vocabulary of {self.vocab_size}")

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

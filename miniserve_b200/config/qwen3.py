"""Typed configuration of the Qwen3 dense decoder, read from config.json keys.

Mirrors the keys the reference reads (miniserve/model/qwen3.py:25-55): the same ten
numbers, ``rope_scaling`` and a non-SiLU ``hidden_act`` rejected, ``head_dim`` defaulting
to hidden_size // num_attention_heads, ``tie_word_embeddings`` defaulting to False.
``max_position_embeddings`` is carried along (the reference never reads it) only to
bound context lengths that the command line may ask for.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    vocab_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int | None = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        if raw.get("rope_scaling"):
            raise NotImplementedError(f"rope_scaling={raw['rope_scaling']!r} is not supported")
        if raw.get("hidden_act", "silu") != "silu":
            raise NotImplementedError(f"hidden_act={raw['hidden_act']!r} is not supported")
        missing = [k for k in ("hidden_size", "intermediate_size", "vocab_size", "num_hidden_layers",
                               "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta")
                   if k not in raw]
        if missing:
            raise KeyError(f"config.json lacks {missing}")
        heads = int(raw["num_attention_heads"])
        cfg = cls(
            hidden_size=int(raw["hidden_size"]),
            intermediate_size=int(raw["intermediate_size"]),
            vocab_size=int(raw["vocab_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=int(raw["num_key_value_heads"]),
            head_dim=int(raw.get("head_dim") or int(raw["hidden_size"]) // heads),
            rms_norm_eps=float(raw["rms_norm_eps"]),
            rope_theta=float(raw["rope_theta"]),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=raw.get("max_position_embeddings"),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("hidden_size", "intermediate_size", "vocab_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ValueError(f"head_dim={self.head_dim} must be even for rotate-half position encoding")
        if not self.rms_norm_eps > 0:
            raise ValueError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")

    def to_dict(self) -> dict[str, Any]:
        """The config.json this configuration would be read from."""
        out = dict(
            architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
            hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            vocab_size=self.vocab_size, num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads, num_key_value_heads=self.num_key_value_heads,
            head_dim=self.head_dim, rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta,
            tie_word_embeddings=self.tie_word_embeddings,
        )
        if self.max_position_embeddings is not None:
            out["max_position_embeddings"] = self.max_position_embeddings
        return out

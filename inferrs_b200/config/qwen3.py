"""Typed configuration of the Qwen3 dense decoder.

Keys and meanings follow the reference's ``to_qwen3_config``
(inferrs-models/src/config.rs:468-502) and ``Qwen3Config``
(inferrs-models/src/models/qwen3.rs:27-45).  The reference falls back to the
sizes of one published checkpoint when a key is absent; here a size that
config.json does not give is an error, so that no model size stands in code.
Only ``head_dim`` keeps its derived default ``hidden_size / num_attention_heads``
(config.rs:487).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, RawConfig


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    # None: config.json does not say; the presence of ``lm_head.weight`` decides,
    # as in the reference (qwen3.rs:366-373).
    tie_word_embeddings: Optional[bool]
    eos_token_ids: Tuple[int, ...] = ()

    REQUIRED_INTS = (
        "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
        "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
    )

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "Qwen3Config":
        missing = [k for k in cls.REQUIRED_INTS + ("rms_norm_eps", "rope_theta") if not raw.has(k)]
        if missing:
            raise ConfigError(f"{raw.source}: Qwen3 config lacks the keys {missing}")
        ints = {k: raw.get_int(k) for k in cls.REQUIRED_INTS}
        for k, v in ints.items():
            if v <= 0:
                raise ConfigError(f"{raw.source}: key '{k}' must be positive, got {v}")
        nh, nkv, hidden = ints["num_attention_heads"], ints["num_key_value_heads"], ints["hidden_size"]
        if raw.has("head_dim"):
            head_dim = raw.get_int("head_dim")
        else:
            if hidden % nh:
                raise ConfigError(
                    f"{raw.source}: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {nh}")
            head_dim = hidden // nh
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"{raw.source}: head_dim must be positive and even (rotary halves), got {head_dim}")
        if nh % nkv:
            raise ConfigError(
                f"{raw.source}: num_attention_heads {nh} is not a multiple of num_key_value_heads {nkv}")
        eps = raw.get_float("rms_norm_eps")
        theta = raw.get_float("rope_theta")
        if not eps > 0.0:
            raise ConfigError(f"{raw.source}: rms_norm_eps must be positive, got {eps}")
        if not theta > 0.0:
            raise ConfigError(f"{raw.source}: rope_theta must be positive, got {theta}")

        # Keys that the reference parses and ignores (config.rs:291-292 and the
        # unused fields of RawConfig).  Where a value would change the arithmetic
        # of the model it is refused instead of being ignored.
        act = raw.get_str("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{raw.source}: hidden_act '{act}' is not supported (the decoder's gate is SiLU)")
        if raw.get_bool("attention_bias", False):
            raise ConfigError(f"{raw.source}: attention_bias=true is not supported (projections have no bias)")
        if raw.has("rope_scaling"):
            raise ConfigError(f"{raw.source}: rope_scaling={raw.values['rope_scaling']!r} is not supported")
        if raw.get_bool("use_sliding_window", False):
            raise ConfigError(f"{raw.source}: use_sliding_window=true is not supported (all layers see all keys)")

        eos: Tuple[int, ...] = ()
        if raw.has("eos_token_id"):
            v = raw.values["eos_token_id"]
            if isinstance(v, int) and not isinstance(v, bool):
                eos = (v,)
            elif isinstance(v, list) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
                eos = tuple(v)
            else:
                raise ConfigError(f"{raw.source}: eos_token_id must be an integer or a list of integers, got {v!r}")
            for t in eos:
                if not 0 <= t < ints["vocab_size"]:
                    raise ConfigError(f"{raw.source}: eos_token_id {t} is outside the vocabulary")

        return cls(
            vocab_size=ints["vocab_size"],
            hidden_size=hidden,
            intermediate_size=ints["intermediate_size"],
            num_hidden_layers=ints["num_hidden_layers"],
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            rms_norm_eps=eps,
            rope_theta=theta,
            max_position_embeddings=ints["max_position_embeddings"],
            tie_word_embeddings=raw.get_bool("tie_word_embeddings", None),
            eos_token_ids=eos,
        )

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        d = {
            "architectures": ["Qwen3ForCausalLM"],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu",
        }
        if self.tie_word_embeddings is not None:
            d["tie_word_embeddings"] = self.tie_word_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

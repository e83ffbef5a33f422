"""Qwen3 dense decoder, written down as a :class:`ModelSpec`.

This file holds no arithmetic.  It says which parts the architecture is made
of, with which tensor names and which config.json values, following the
reference model (inferrs-models/src/models/qwen3.rs):

* tensors live under ``model.`` (qwen3.rs:343); projections have no bias
  (qwen3.rs:76-79); per-head RMSNorm on queries and keys with the layer norms'
  eps (qwen3.rs:80-81); rotation over the whole head with ``rope_theta``
  (qwen3.rs:375-385); score scale 1/sqrt(head_dim) (qwen3.rs:165-175);
* pre-norm residual block (qwen3.rs:285-300) with a SiLU-gated feed-forward
  (inferrs-models/src/models/attention_utils.rs:94-118);
* final norm, then the head; the embedding table stands in for an absent
  ``lm_head.weight`` (qwen3.rs:364-373).
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.qwen3 import Qwen3Config
from ..parts.spec import (AttentionSpec, GatedDenseSpec, ModelSpec, NormSpec, PositionSpec, default_schedule,
                          pre_norm_layer)

ARCHITECTURE = "Qwen3ForCausalLM"


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    position = PositionSpec(kind="rotary_split_half", rot_dim=cfg.head_dim, theta=cfg.rope_theta,
                            max_positions=cfg.max_position_embeddings)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        attn = AttentionSpec(
            width=cfg.hidden_size,
            n_heads=cfg.num_attention_heads,
            n_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim,
            scale=1.0 / math.sqrt(cfg.head_dim),
            position=position,
            q_proj=f"{p}.self_attn.q_proj.weight",
            k_proj=f"{p}.self_attn.k_proj.weight",
            v_proj=f"{p}.self_attn.v_proj.weight",
            o_proj=f"{p}.self_attn.o_proj.weight",
            q_norm=NormSpec(size=cfg.head_dim, eps=cfg.rms_norm_eps, weight=f"{p}.self_attn.q_norm.weight"),
            k_norm=NormSpec(size=cfg.head_dim, eps=cfg.rms_norm_eps, weight=f"{p}.self_attn.k_norm.weight"),
            window=None,
        )
        ffn = GatedDenseSpec(
            width=cfg.hidden_size,
            inner=cfg.intermediate_size,
            gate_proj=f"{p}.mlp.gate_proj.weight",
            up_proj=f"{p}.mlp.up_proj.weight",
            down_proj=f"{p}.mlp.down_proj.weight",
            activation="silu",
        )
        layers.append(pre_norm_layer(
            mixer_norm=NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps, weight=f"{p}.input_layernorm.weight"),
            mixer=attn,
            ffn_norm=NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps,
                              weight=f"{p}.post_attention_layernorm.weight"),
            ffn=ffn,
        ))
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        width=cfg.hidden_size,
        embedding="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=default_schedule(cfg.num_hidden_layers),
        final_norm=NormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps, weight="model.norm.weight"),
        lm_head="lm_head.weight",
        # config.json says "untied": the head must be there.  Otherwise its
        # presence decides, as in the reference.
        lm_head_optional=cfg.tie_word_embeddings is not False,
        max_positions=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_token_ids,
        architecture=ARCHITECTURE,
    )


register_architecture(ARCHITECTURE, Qwen3Config, build_spec, model_type="qwen3", replace=True)

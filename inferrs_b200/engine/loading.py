"""From a model folder (config.json + safetensors) to a description and weights on the device.

Mirrors the reference's load path (inferrs/src/engine.rs:104-207): read config.json, detect the
architecture, build its typed configuration, then load tensors by name.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.base import RawConfig, resolve_architecture
from ..parts.spec import ModelSpec
from ..runtime import Runtime
from ..weights.loader import load_weights
from ..weights.random_init import random_weights
from .model import declared_tensors


def spec_from_config(config) -> Tuple[ModelSpec, object]:
    """(model description, typed configuration) from a config.json path, folder or dict."""
    raw = config if isinstance(config, RawConfig) else (
        RawConfig(config, "<dict>") if isinstance(config, dict) else RawConfig.from_file(config))
    arch = resolve_architecture(raw)
    cfg = arch.config_cls.from_raw(raw)
    return arch.build_spec(cfg), cfg


def load_model_dir(model_dir: str, rt: Runtime) -> Tuple[ModelSpec, Dict[str, torch.Tensor], object]:
    spec, cfg = spec_from_config(model_dir)
    weights = load_weights(model_dir, declared_tensors(spec), rt.dtype, rt.device)
    return spec, weights, cfg


def random_model(config: dict, seed: int, rt: Runtime, tied: bool = None
                 ) -> Tuple[ModelSpec, Dict[str, torch.Tensor], object]:
    """Random weights made directly on the device (no files), for sizes too large to write out."""
    spec, cfg = spec_from_config(config)
    if tied is None:
        tied = bool(config.get("tie_word_embeddings", False))
    weights = random_weights(declared_tensors(spec), seed, rt.dtype, rt.device, skip_optional=tied)
    return spec, weights, cfg

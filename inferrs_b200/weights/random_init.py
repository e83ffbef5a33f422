"""Random weights from a configuration and a seed.

The reference has no such mode (its tests need downloaded checkpoints,
inferrs/tests/server_integration.rs); it exists here so that every size of the
architecture can be run without one.  Matrices and the embedding table are
N(0, 0.02); norm weights are 1 + U(-0.1, 0.1), so that a kernel that forgets a
norm weight does not pass by accident.  Each tensor has a generator of its own,
seeded from the seed and the tensor's place in the model's declaration, so a
tensor's values do not depend on which other tensors are made.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Optional

import torch

from ..config.base import RawConfig, resolve_architecture
from ..parts.spec import TensorDecl
from .safetensors_io import write_safetensors

NORMAL_STD = 0.02
NORM_SPREAD = 0.1


def random_tensor(decl: TensorDecl, index: int, seed: int, dtype: torch.dtype,
                  device: torch.device = torch.device("cpu")) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1_000_003 + index * 7919 + 12345) % (2 ** 63 - 1))
    if decl.init == "normal":
        t = torch.empty(decl.shape, dtype=torch.float32, device=device).normal_(0.0, NORMAL_STD, generator=g)
    elif decl.init == "norm":
        t = torch.empty(decl.shape, dtype=torch.float32, device=device).uniform_(-NORM_SPREAD, NORM_SPREAD,
                                                                                 generator=g)
        t += 1.0
    else:
        raise ValueError(f"tensor '{decl.name}': unknown init '{decl.init}'")
    return t.to(dtype)


def random_weights(decls: Iterable[TensorDecl], seed: int, dtype: torch.dtype,
                   device: torch.device = torch.device("cpu"), skip_optional: bool = False
                   ) -> Dict[str, torch.Tensor]:
    """All declared tensors, made on ``device`` (values differ between devices)."""
    out: Dict[str, torch.Tensor] = {}
    for i, d in enumerate(decls):
        if d.name in out or (d.optional and skip_optional):
            continue
        out[d.name] = random_tensor(d, i, seed, dtype, device)
    return out


def write_random_model(model_dir: str, config: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       tied: Optional[bool] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``model_dir``.

    ``tied``: leave the optional head tensor out (True) or write it (False);
    by default it is left out exactly when config.json says
    ``tie_word_embeddings: true``.
    """
    from .. import models  # noqa: F401  (registers the architectures)
    from ..engine.model import declared_tensors  # late: engine imports weights

    raw = RawConfig(config, source="<random model>")
    arch = resolve_architecture(raw)
    cfg = arch.config_cls.from_raw(raw)
    spec = arch.build_spec(cfg)
    if tied is None:
        tied = bool(config.get("tie_word_embeddings", False))
    decls = declared_tensors(spec)
    weights = random_weights(decls, seed, dtype, skip_optional=tied)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), weights.items(),
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir

"""Random weights from a configuration and a seed.

The reference has no such mode (its tests need downloaded checkpoints,
inferrs/tests/server_integration.rs); it exists here so that every size of the
architecture can be run without one.  Matrices and the embedding table are
N(0, 0.02) (a sum of twelve uniform 16-bit numbers stands in for the normal law:
its tails end at six standard deviations); norm weights are 1 + U(-0.1, 0.1), so
that a kernel that forgets a norm weight does not pass by accident.

A value depends on the seed, the tensor's name and the element's index and on
nothing else: it is made by integer arithmetic on the index (a 64-bit mixing
function), which gives the same bits on the host and on the device, in any
order and in pieces of any size.  So a model folder written from a seed and a
model made on the device from the same seed hold the same weights.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Optional

import torch

from ..config.base import RawConfig, resolve_architecture
from ..parts.spec import TensorDecl
from .safetensors_io import write_safetensors_streamed

NORMAL_STD = 0.02
NORM_SPREAD = 0.1
_CHUNK = 1 << 22          # elements made at a time (the 64-bit intermediates of a large table would not fit beside it)
_MASK64 = (1 << 64) - 1


def _i64(v: int) -> int:
    """An unsigned 64-bit number as the signed one with the same bits."""
    v &= _MASK64
    return v - (1 << 64) if v >= (1 << 63) else v


_GOLDEN = _i64(0x9E3779B97F4A7C15)
_M1 = _i64(0xBF58476D1CE4E5B9)
_M2 = _i64(0x94D049BB133111EB)


def _lsr(x: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 bit patterns."""
    return (x >> n) & ((1 << (64 - n)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    """The finishing function of splitmix64 on int64 tensors (products wrap, as unsigned ones do)."""
    x = (x ^ _lsr(x, 30)) * _M1
    x = (x ^ _lsr(x, 27)) * _M2
    return x ^ _lsr(x, 31)


def _mix_int(v: int) -> int:
    v &= _MASK64
    v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & _MASK64
    return v ^ (v >> 31)


def _tensor_key(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325                       # FNV-1a over the name
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _MASK64
    return _mix_int(_mix_int(int(seed)) ^ h)


def _fill(out: torch.Tensor, key: int, init: str):
    flat = out.view(-1)
    n = flat.shape[0]
    for start in range(0, n, _CHUNK):
        stop = min(n, start + _CHUNK)
        idx = torch.arange(start, stop, dtype=torch.int64, device=out.device)
        if init == "normal":
            total = torch.zeros(stop - start, dtype=torch.int64, device=out.device)
            for k in range(3):                   # three 64-bit numbers: twelve 16-bit ones
                h = _mix((idx * 3 + k) * _GOLDEN + _i64(key))
                for shift in (0, 16, 32, 48):
                    total += _lsr(h, shift) & 0xFFFF
            # mean 12 * 32767.5, standard deviation 65536 (to three parts in ten thousand million)
            z = (total - 393210).to(torch.float32) * (1.0 / 65536.0)
            flat[start:stop] = z * NORMAL_STD
        else:
            h = _mix(idx * _GOLDEN + _i64(key))
            u = (_lsr(h, 40)).to(torch.float32) * (1.0 / 16777216.0)          # 24 bits: [0, 1)
            flat[start:stop] = (u * 2.0 - 1.0) * NORM_SPREAD + 1.0


def random_tensor(decl: TensorDecl, index: int, seed: int, dtype: torch.dtype,
                  device: torch.device = torch.device("cpu")) -> torch.Tensor:
    """``index`` (the tensor's place in the declaration) plays no part: the name does."""
    if decl.init not in ("normal", "norm"):
        raise ValueError(f"tensor '{decl.name}': unknown init '{decl.init}'")
    t = torch.empty(decl.shape, dtype=torch.float32, device=device)
    _fill(t, _tensor_key(seed, decl.name), decl.init)
    return t.to(dtype)


def random_weights(decls: Iterable[TensorDecl], seed: int, dtype: torch.dtype,
                   device: torch.device = torch.device("cpu"), skip_optional: bool = False
                   ) -> Dict[str, torch.Tensor]:
    """All declared tensors, made on ``device`` (the same values on every device)."""
    out: Dict[str, torch.Tensor] = {}
    for i, d in enumerate(decls):
        if d.name in out or (d.optional and skip_optional):
            continue
        out[d.name] = random_tensor(d, i, seed, dtype, device)
    return out


def write_random_model(model_dir: str, config: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       tied: Optional[bool] = None, device: Optional[torch.device] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``model_dir``.

    ``tied``: leave the optional head tensor out (True) or write it (False);
    by default it is left out exactly when config.json says
    ``tie_word_embeddings: true``.  The tensors are made one at a time, on ``device`` (by default the GPU if there
    is one: the same bits as on the host, a hundred times as fast), and written as they come, so the folder of a
    model larger than the host's memory can be written.
    """
    from .. import models  # noqa: F401  (registers the architectures)
    from ..engine.model import declared_tensors  # late: engine imports weights

    raw = RawConfig(config, source="<random model>")
    arch = resolve_architecture(raw)
    cfg = arch.config_cls.from_raw(raw)
    spec = arch.build_spec(cfg)
    if tied is None:
        tied = bool(config.get("tie_word_embeddings", False))
    if device is None:
        device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    entries, seen = [], set()
    for i, d in enumerate(declared_tensors(spec)):
        if d.name in seen or (d.optional and tied):
            continue
        seen.add(d.name)
        entries.append((d.name, tuple(d.shape), dtype, (lambda d=d, i=i: random_tensor(d, i, seed, dtype, device))))
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=1)
    write_safetensors_streamed(os.path.join(model_dir, "model.safetensors"), entries,
                               metadata={"format": "pt", "seed": str(seed)})
    return model_dir

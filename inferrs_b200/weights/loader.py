"""Weights by tensor name, checked against what the model's parts declare.

The reference looks every tensor up by its dotted name, checks its shape and
casts it to the run dtype (candle-nn/src/var_builder.rs:186-192, :501-520), and
takes ``model.safetensors`` or else all ``*.safetensors`` sorted by name, a
later file winning on duplicates (inferrs/src/hub.rs:54-75,
candle-core/src/safetensors.rs:454-480).  It stops at the first tensor that is
missing.  Here all names and shapes are compared before a byte is read, and
one :class:`WeightError` lists everything that is missing, unexpected or of the
wrong shape.

Precision rule: with ``dtype=float32`` every floating tensor becomes float32.
With ``dtype=bfloat16`` a tensor stored in bfloat16 stays bfloat16, a tensor
stored in float32 stays float32 (the parts run such a tensor through their
32-bit kernels), float16 becomes bfloat16; integer tensors become int32.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from ..parts.spec import TensorDecl
from .safetensors_io import SafetensorsError, SafetensorsFile, TensorInfo

_FLOATS = ("F32", "F16", "BF16", "F64")
_INTS = ("I64", "I32", "I16", "I8", "U8")


class WeightError(ValueError):
    """The weight files do not hold what the model needs.

    ``missing``, ``unexpected`` and ``wrong_shape`` carry the findings; the
    message lists all of them.
    """

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[str], other: Sequence[str] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        if self.other:
            lines.append("  " + "; ".join(self.other))
        super().__init__("\n".join(lines))


def weight_files(model_dir: str) -> List[str]:
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise WeightError(model_dir, [], [], [], [f"no model.safetensors and no *.safetensors in {model_dir}"])
    return files


def convert_for(t: torch.Tensor, stored: str, dtype: torch.dtype) -> torch.Tensor:
    """Apply the precision rule of this module to one tensor."""
    if stored in _INTS:
        return t.to(torch.int32)
    if dtype == torch.float32:
        return t.to(torch.float32)
    if dtype == torch.bfloat16:
        if stored in ("F32", "BF16"):
            return t
        if stored == "F64":
            return t.to(torch.float32)
        return t.to(torch.bfloat16)
    raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")


def check_declared(where: str, decls: Iterable[TensorDecl], present: Dict[str, TensorInfo]):
    """Raise one WeightError for everything that does not match; return the names to read."""
    missing, wrong, other = [], [], []
    wanted = {}
    for d in decls:
        if d.name in wanted:
            if wanted[d.name].shape != tuple(d.shape):
                other.append(f"{d.name} is declared twice with shapes {list(wanted[d.name].shape)} and {list(d.shape)}")
            continue
        wanted[d.name] = d
        if d.name not in present:
            if not d.optional:
                missing.append(d.name)
            continue
        ti = present[d.name]
        if tuple(ti.shape) != tuple(d.shape):
            wrong.append(f"{d.name}: expected {list(d.shape)}, found {list(ti.shape)}")
        if ti.dtype not in _FLOATS and ti.dtype not in _INTS:
            other.append(f"{d.name}: dtype {ti.dtype} is not supported")
    unexpected = sorted(n for n in present if n not in wanted)
    if missing or unexpected or wrong or other:
        raise WeightError(where, missing, unexpected, wrong, other)
    return [n for n in wanted if n in present]


def load_weights(model_dir: str, decls: Iterable[TensorDecl], dtype: torch.dtype,
                 device: Optional[torch.device] = None) -> Dict[str, torch.Tensor]:
    """Read every declared tensor, by name, into ``device`` memory."""
    decls = list(decls)
    files = []
    try:
        for p in weight_files(model_dir):
            files.append(SafetensorsFile(p))
    except SafetensorsError as e:
        raise WeightError(model_dir, [], [], [], [str(e)]) from e
    try:
        present: Dict[str, TensorInfo] = {}
        owner: Dict[str, SafetensorsFile] = {}
        for f in files:  # a later file wins
            for name, ti in f.info.items():
                present[name] = ti
                owner[name] = f
        names = check_declared(model_dir, decls, present)
        out: Dict[str, torch.Tensor] = {}
        # for another device the bytes go there straight from the mapped file (the copy is done when .to() returns)
        elsewhere = device is not None and torch.device(device).type != "cpu"
        t = None
        for name in names:
            t = convert_for(owner[name].read(name, private=not elsewhere), present[name].dtype, dtype)
            if device is not None:
                t = t.to(device)
            out[name] = t
        del t
        return out
    finally:
        for f in files:
            f.close()

"""Where and in which precision a model runs."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict

import torch

_DTYPE_NAMES = {
    "float32": torch.float32, "f32": torch.float32, "fp32": torch.float32,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
}


def parse_dtype(name) -> torch.dtype:
    """``bfloat16``/``bf16`` or ``float32``/``f32`` (the reference's ``--dtype`` spellings, inferrs/src/main.rs:101-103;
    float16 is not offered here)."""
    if isinstance(name, torch.dtype):
        if name in (torch.float32, torch.bfloat16):
            return name
        raise ValueError(f"dtype must be float32 or bfloat16, got {name}")
    try:
        return _DTYPE_NAMES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPE_NAMES)}, got {name!r}") from None


@dataclass
class Runtime:
    """``dtype`` is the element type of activations and of the cache.  The residual stream,
    norms, softmax, rotation and logits are float32 in both cases; with float32 every matrix
    product is true 32-bit as well."""

    device: torch.device
    dtype: torch.dtype
    shared: Dict[Any, Any] = field(default_factory=dict)  # tables shared by parts with equal descriptions

    @classmethod
    def cuda(cls, dtype) -> "Runtime":
        if not torch.cuda.is_available():
            raise RuntimeError("inferrs_b200 needs a CUDA device (built for sm_100a); there is no CPU path")
        return cls(device=torch.device("cuda", torch.cuda.current_device()), dtype=parse_dtype(dtype))

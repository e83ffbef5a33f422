"""How a layer's two sub-layers and their norms are arranged around the residual stream."""
from __future__ import annotations

from typing import Optional

import torch

from .registry import register_arrangement


class PreNormBlock:
    """x += mixer(norm(x)); x += feed_forward(norm(x))  (inferrs-models/src/models/qwen3.rs:285-300).

    The residual stream ``x`` is float32 and is updated in place.  An addition is not done where
    the sub-layer ends but inside the norm kernel that follows it, so the block hands its last
    sub-layer's output on as ``pending`` and takes the previous block's in.
    """

    def __init__(self, spec, mixer_norm, mixer, ffn_norm, ffn):
        self.spec = spec
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def forward(self, ctx, cache_id: int, residual: torch.Tensor, pending: Optional[torch.Tensor]) -> torch.Tensor:
        h = self.mixer_norm.add_norm(residual, pending)
        a = self.mixer.forward(ctx, cache_id, h)
        h = self.ffn_norm.add_norm(residual, a)
        return self.ffn.forward(ctx, h)


register_arrangement("pre_norm", PreNormBlock)

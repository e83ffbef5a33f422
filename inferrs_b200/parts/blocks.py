"""How a layer's sub-layers and their norms are arranged around the residual stream."""
from __future__ import annotations

from typing import List, Optional

import torch

from .registry import register_arrangement


class BuiltSubLayer:
    """A sub-layer whose parts are built: ``part`` with its ``category`` ("mixer" or "feed_forward"),
    the ``norm`` before it and the ``post_norm`` after it (either may be None)."""

    def __init__(self, category: str, part, norm=None, post_norm=None):
        self.category, self.part, self.norm, self.post_norm = category, part, norm, post_norm

    def run(self, ctx, cache_id: int, h: torch.Tensor) -> torch.Tensor:
        y = self.part.forward(ctx, cache_id, h) if self.category == "mixer" else self.part.forward(ctx, h)
        return self.post_norm.norm(y) if self.post_norm is not None else y


class SequentialBlock:
    """For every sub-layer in turn: x += post_norm(part(norm(x))).  With two sub-layers, a mixer and a
    feed-forward with a norm each, this is the reference's decoder layer
    (inferrs-models/src/models/qwen3.rs:285-300).

    The residual stream ``x`` is float32 and is updated in place.  An addition is not done where
    the sub-layer ends but inside the norm kernel that follows it, so the block hands its last
    sub-layer's output on as ``pending`` and takes the previous block's in.
    """

    def __init__(self, spec, sublayers: List[BuiltSubLayer]):
        if not sublayers:
            raise ValueError("a layer needs at least one sub-layer")
        if any(s.norm is None for s in sublayers):
            # the output of the sub-layer before is added inside the norm kernel: "no norm" is a part too
            raise ValueError("every sub-layer of a sequential block needs a norm part (NoNorm where there is none)")
        self.spec = spec
        self.sublayers = list(sublayers)

    def parts(self):
        """Every part of the block (the runner asks each whether it is ``graph_safe``)."""
        for s in self.sublayers:
            yield s.part
            if s.norm is not None:
                yield s.norm
            if s.post_norm is not None:
                yield s.post_norm

    def forward(self, ctx, cache_id: int, residual: torch.Tensor, pending: Optional[torch.Tensor]) -> torch.Tensor:
        for s in self.sublayers:
            h = s.norm.add_norm(residual, pending)
            pending = s.run(ctx, cache_id, h)
        return pending


register_arrangement("sequential", SequentialBlock)

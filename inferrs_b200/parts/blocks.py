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

    def run(self, ctx, cache_id: int, h, sink=None):
        kw = {} if sink is None else {"sink": sink}
        y = self.part.forward(ctx, cache_id, h, **kw) if self.category == "mixer" else self.part.forward(ctx, h, **kw)
        return self.post_norm.norm(y) if self.post_norm is not None else y

    def takes_scaled_rows(self, n_rows: int) -> bool:
        """Whether this sub-layer can be handed scaled rows in place of its norm's output: the norm must be able to
        give a sink to the product before it, and the part must say that it reads scaled rows."""
        f = getattr(self.part, "takes_scaled_rows", None)
        return f is not None and hasattr(self.norm, "sink") and bool(f(n_rows))

    def feeds_sink(self, n_rows: int) -> bool:
        f = getattr(self.part, "feeds_sink", None)
        return f is not None and self.post_norm is None and bool(f(n_rows))


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

    def entry(self) -> BuiltSubLayer:
        """The sub-layer that takes what the block before hands on."""
        return self.sublayers[0]

    def forward(self, ctx, cache_id: int, residual: torch.Tensor, pending, after: Optional[BuiltSubLayer] = None):
        """``after``: the sub-layer that runs after this block (the next block's entry), if the caller knows it.  Where
        a sub-layer's last product and the next sub-layer's first both fold norms at this step's number of rows,
        the addition to the residual stream and the norm between them run inside the two products: the producer gets
        the norm's sink and hands on scaled rows, which the norm passes through."""
        n_rows = residual.shape[0]
        for i, s in enumerate(self.sublayers):
            h = s.norm.add_norm(residual, pending)
            nxt = self.sublayers[i + 1] if i + 1 < len(self.sublayers) else after
            fold = nxt is not None and s.feeds_sink(n_rows) and nxt.takes_scaled_rows(n_rows)
            pending = s.run(ctx, cache_id, h, sink=nxt.norm.sink(residual) if fold else None)
        return pending


register_arrangement("sequential", SequentialBlock)

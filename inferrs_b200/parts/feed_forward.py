"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..runtime import Runtime
from .basic import Linear, fuse_rows
from .registry import register_feed_forward
from .spec import GatedDenseSpec, TensorDecl


class GatedDense:
    """down( silu(gate(x)) * up(x) ), silu(z) = z / (1 + exp(-z))
    (inferrs-models/src/models/attention_utils.rs:94-118; inferrs-kernels/candle-kernels/src/unary.cu:58-61).
    Gate and up weights are stacked at load: one product feeds the gate kernel, or, for a few rows, one
    kernel does both products and the gate."""

    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def declare(spec: GatedDenseSpec) -> List[TensorDecl]:
        return [TensorDecl(spec.gate_proj, (spec.inner, spec.width)),
                TensorDecl(spec.up_proj, (spec.inner, spec.width)),
                TensorDecl(spec.down_proj, (spec.width, spec.inner))]

    def __init__(self, spec: GatedDenseSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.activation != "silu":
            raise ValueError(f"gated feed-forward: activation '{spec.activation}' has no kernel (only 'silu')")
        self.spec = spec
        self.rt = rt
        self.gate_up = Linear(fuse_rows([weights[spec.gate_proj], weights[spec.up_proj]]), rt)
        self.down = Linear(weights[spec.down_proj], rt)

    def takes_scaled_rows(self, n_rows: int) -> bool:
        return self.gate_up.folds_norms(n_rows) and n_rows <= kernels.SWIGLU_MAX_TOKENS

    def feeds_sink(self, n_rows: int) -> bool:
        return self.down.folds_norms(n_rows)

    def forward(self, ctx, h, sink=None):
        a = torch.empty((h.shape[0], self.spec.inner), dtype=self.rt.dtype, device=h.device)
        kernels.gated_linear(h, self.gate_up.weight, a, self.rt.dtype)
        return self.down(a, sink=sink)


register_feed_forward("gated_dense", GatedDense)

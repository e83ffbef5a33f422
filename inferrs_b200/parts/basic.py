"""Norm, position encoding and the matrix product that the other parts are made of."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels
from ..runtime import Runtime
from .registry import register_norm, register_position
from .spec import NormSpec, PositionSpec, TensorDecl


class RMSNorm:
    """x / sqrt(mean(x^2) + eps) * w, in float32 (inferrs-kernels/candle-kernels/src/reduce.cu:188-228),
    fused with the residual addition that precedes it in a block."""

    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def declare(spec: NormSpec) -> List[TensorDecl]:
        return [TensorDecl(spec.weight, (spec.size,), init="norm")]

    def __init__(self, spec: NormSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = weights[spec.weight]

    def add_norm(self, residual: torch.Tensor, delta, rows: Optional[torch.Tensor] = None):
        if isinstance(delta, kernels.ScaledRows):
            # the product before has added its result to the residual stream and folded this norm in (it was given
            # this norm's sink): what it handed on stands for the norm's output
            if rows is not None:
                raise ValueError("scaled rows stand for all rows of a step, not for a choice of them")
            return delta
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.rt.dtype, device=residual.device)
        kernels.add_rms_norm(residual, delta, self.weight, self.spec.eps, out, rows)
        return out

    def sink(self, residual: torch.Tensor) -> "kernels.ResidualSink":
        """For a product that can fold the addition to the residual stream and this norm into its read-back."""
        return kernels.ResidualSink(residual, self.weight, self.spec.eps)

    def norm(self, x: torch.Tensor) -> torch.Tensor:
        """The norm alone, on rows in the activation dtype (a norm on a sub-layer's output)."""
        out = torch.empty_like(x)
        kernels.rms_norm_rows(x, self.weight, self.spec.eps, out)
        return out


class NoNorm:
    """No norm: the sub-layer reads (or hands on) the rows as they are.  Still the place where the output of
    the sub-layer before it is added to the residual stream."""

    graph_safe = True

    @staticmethod
    def declare(spec) -> List[TensorDecl]:
        return []

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, residual.shape[1]), dtype=self.rt.dtype, device=residual.device)
        kernels.add_cast(residual, delta, out, rows)
        return out

    def norm(self, x: torch.Tensor) -> torch.Tensor:
        return x


register_norm("rms", RMSNorm)
register_norm("none", NoNorm)


class RotarySplitHalf:
    """cos/sin of position * theta^(-2i/rot_dim), i < rot_dim/2, all in float32
    (inferrs-models/src/models/attention_utils.rs:186-216); element i is rotated with
    element i + rot_dim/2 (attention_utils.rs:137-151).  The reference casts the tables to the
    run dtype; here they stay float32."""

    def __init__(self, spec: PositionSpec, rt: Runtime):
        if spec.rot_dim <= 0 or spec.rot_dim % 2:
            raise ValueError(f"rot_dim must be positive and even, got {spec.rot_dim}")
        if spec.max_positions <= 0:
            raise ValueError(f"max_positions must be positive, got {spec.max_positions}")
        self.spec = spec
        half = spec.rot_dim // 2
        exponent = torch.arange(half, dtype=torch.float32) * 2.0 / float(spec.rot_dim)
        inv_freq = 1.0 / torch.pow(torch.tensor(float(spec.theta), dtype=torch.float32), exponent)
        angle = torch.arange(spec.max_positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
        self.cos = torch.cos(angle).contiguous().to(rt.device)
        self.sin = torch.sin(angle).contiguous().to(rt.device)

    def tables(self):
        return self.cos, self.sin, self.spec.rot_dim


class RotaryInterleaved(RotarySplitHalf):
    """The same tables; element 2i of a head is rotated with element 2i + 1."""

    interleaved = True


class NoPosition:
    def __init__(self, spec: PositionSpec, rt: Runtime):
        self.spec = spec

    def tables(self):
        return None, None, 0


register_position("rotary_split_half", RotarySplitHalf)
register_position("rotary_interleaved", RotaryInterleaved)
register_position("none", NoPosition)


def build_position(spec: PositionSpec, rt: Runtime):
    """One table per distinct description, shared by all layers that name it."""
    from .registry import part_class

    key = ("position", spec)
    if key not in rt.shared:
        rt.shared[key] = part_class("position", spec)(spec, rt)
    return rt.shared[key]


def fuse_rows(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """Stack weight matrices [out_i, in] along ``out``.  Mixed precisions become float32."""
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(list(tensors), dim=0).contiguous()


class Linear:
    """y = x W^T, W stored [out, in], no bias (candle-nn/src/linear.rs:41-82).

    float32 runs: FFMA kernel.  bfloat16 runs: tensor-core product with float32 accumulation for a
    bfloat16 weight; a weight that is stored in float32 keeps its precision and goes through the
    FFMA kernel with the bfloat16 activations widened on the fly.
    """

    def __init__(self, weight: torch.Tensor, rt: Runtime):
        if weight.dim() != 2:
            raise ValueError(f"a linear weight must be a matrix, got shape {tuple(weight.shape)}")
        self.weight = weight.contiguous()
        self.rt = rt
        self.n_out, self.n_in = weight.shape

    def __call__(self, x, out_dtype: Optional[torch.dtype] = None, sink=None):
        """``x`` may be :class:`~inferrs_b200.kernels.ScaledRows`; with a ``sink`` the result is added to the residual
        stream there and the next norm's scaled rows come back instead of the result."""
        out = torch.empty((x.shape[0], self.n_out), dtype=out_dtype or self.rt.dtype, device=x.device)
        scaled = kernels.linear(x, self.weight, out, self.rt.dtype, sink=sink)
        return out if sink is None else scaled

    def folds_norms(self, n_rows: int) -> bool:
        """Whether this product takes scaled rows and feeds a sink at this number of rows."""
        return kernels.folded_norm_supported(n_rows, self.rt.dtype, self.weight)

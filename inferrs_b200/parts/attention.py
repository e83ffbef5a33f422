"""Grouped-query attention over the paged cache.

The arithmetic is the reference's (inferrs-models/src/models/qwen3.rs:104-196):
project, split into heads, RMSNorm per head on queries and keys, rotate by
position, append keys and values to the cache, scores * scale, causal mask,
softmax, weighted sum of values, output projection.  The reference gathers the
whole context and builds the score matrix with library calls
(inferrs-models/src/models/attention_utils.rs:299-370); here two kernels do it:
one turns the fused projection into rotated queries and writes keys and values
into their pages, one attends over the pages.

Every size is a field of the description; the part does not know which model
or which layer it is in.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.storage import KVNeed
from ..runtime import Runtime
from .basic import Linear, build_position, fuse_rows
from .registry import register_mixer
from .spec import AttentionSpec, TensorDecl


class Attention:
    graph_safe = True  # launches depend only on shapes, never on the step's host-side values

    @staticmethod
    def declare(spec: AttentionSpec) -> List[TensorDecl]:
        d = [TensorDecl(spec.q_proj, (spec.n_heads * spec.head_dim, spec.width)),
             TensorDecl(spec.o_proj, (spec.width, spec.n_heads * spec.head_dim))]
        if spec.own_kv:
            d += [TensorDecl(spec.k_proj, (spec.n_kv_heads * spec.head_dim, spec.width)),
                  TensorDecl(spec.v_proj, (spec.n_kv_heads * spec.head_dim, spec.width))]
        if spec.q_norm is not None:
            d.append(TensorDecl(spec.q_norm.weight, (spec.head_dim,), init="norm"))
        if spec.k_norm is not None and spec.own_kv:
            d.append(TensorDecl(spec.k_norm.weight, (spec.head_dim,), init="norm"))
        return d

    @staticmethod
    def cache_need(spec: AttentionSpec) -> Optional[KVNeed]:
        return KVNeed(n_kv_heads=spec.n_kv_heads, head_dim=spec.head_dim, window=spec.window)

    @staticmethod
    def state_need(spec: AttentionSpec):
        return None

    @staticmethod
    def writes_cache(spec: AttentionSpec) -> bool:
        return spec.own_kv

    def __init__(self, spec: AttentionSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} key/value heads")
        if spec.own_kv and (spec.k_proj is None or spec.v_proj is None):
            raise ValueError("an attention layer with its own keys and values needs k_proj and v_proj")
        for n in (spec.q_norm, spec.k_norm):
            if n is not None and (n.kind != "rms" or n.size != spec.head_dim):
                raise ValueError(f"per-head norm must be an RMS norm over head_dim={spec.head_dim}, got {n}")
        if spec.q_norm is not None and spec.k_norm is not None and spec.q_norm.eps != spec.k_norm.eps:
            raise ValueError("query and key norms must share eps")
        self.spec = spec
        self.rt = rt
        mats = [weights[spec.q_proj]]
        if spec.own_kv:
            mats += [weights[spec.k_proj], weights[spec.v_proj]]
        self.qkv = Linear(fuse_rows(mats), rt)
        self.o = Linear(weights[spec.o_proj], rt)
        self.q_weight = weights[spec.q_norm.weight] if spec.q_norm is not None else None
        self.k_weight = weights[spec.k_norm.weight] if (spec.k_norm is not None and spec.own_kv) else None
        if self.q_weight is not None and self.k_weight is not None and self.q_weight.dtype != self.k_weight.dtype:
            self.q_weight, self.k_weight = self.q_weight.float(), self.k_weight.float()
        self.eps = (spec.q_norm or spec.k_norm).eps if (spec.q_norm or spec.k_norm) else 0.0
        position = build_position(spec.position, rt)
        self.cos, self.sin, self.rot_dim = position.tables()
        self.interleaved = bool(getattr(position, "interleaved", False))   # which elements of a head turn together
        if self.rot_dim > spec.head_dim:
            raise ValueError(f"rot_dim {self.rot_dim} exceeds head_dim {spec.head_dim}")

    # A block may hand this part scaled rows instead of a norm's output, and a sink instead of taking its result, where
    # both of its products fold norms at the step's number of rows (see SequentialBlock).
    def takes_scaled_rows(self, n_rows: int) -> bool:
        return self.qkv.folds_norms(n_rows)

    def feeds_sink(self, n_rows: int) -> bool:
        return self.o.folds_norms(n_rows)

    def forward(self, ctx, cache_id: int, h, sink=None):
        s = self.spec
        n = h.shape[0]
        qkv = self.qkv(h)
        k_pages, v_pages, group = ctx.storage.pages(cache_id)
        table = ctx.block_tables[group]
        q = torch.empty((n, s.n_heads, s.head_dim), dtype=self.rt.dtype, device=h.device)
        kernels.qk_norm_rope_store(qkv, s.n_heads, s.n_kv_heads, s.head_dim, s.own_kv, self.q_weight, self.k_weight,
                                   self.eps, self.cos, self.sin, self.rot_dim, ctx.positions, ctx.row_request,
                                   table, k_pages, v_pages, q, interleaved=self.interleaved)
        out = torch.empty((n, s.n_heads * s.head_dim), dtype=self.rt.dtype, device=h.device)
        kernels.paged_attention(q, k_pages, v_pages, table, ctx, s.scale, s.window, out)
        return self.o(out, sink=sink)


register_mixer("attention", Attention)

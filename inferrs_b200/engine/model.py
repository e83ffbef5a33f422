"""A model assembled from a :class:`ModelSpec`: embedding, scheduled layers, last norm, head.

Nothing here is specific to an architecture.  The reference's counterpart is
``Qwen3Model::forward`` (inferrs-models/src/models/qwen3.rs:398-407): embed,
run the layers, norm, and logits for the rows that are wanted (the reference
wants only the last, inferrs-models/src/models/attention_utils.rs:382-395).
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.storage import KVNeed, StateNeed
from ..parts.basic import Linear, NoNorm
from ..parts.blocks import BuiltSubLayer
from ..parts.registry import part_class
from ..parts.spec import ModelSpec, TensorDecl
from ..runtime import Runtime


class ModelError(ValueError):
    pass


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    """Every tensor the model's parts expect, in a fixed order, each name once."""
    decls: List[TensorDecl] = [TensorDecl(spec.embedding, (spec.vocab_size, spec.width))]
    for layer in spec.layers:
        for sub in layer.sublayers:
            _check_category(sub.category)
            if sub.norm is not None:
                decls += part_class("norm", sub.norm).declare(sub.norm)
            decls += part_class(sub.category, sub.part).declare(sub.part)
            if sub.post_norm is not None:
                decls += part_class("norm", sub.post_norm).declare(sub.post_norm)
    decls += part_class("norm", spec.final_norm).declare(spec.final_norm)
    decls.append(TensorDecl(spec.lm_head, (spec.vocab_size, spec.width), optional=spec.lm_head_optional))
    seen, out = {}, []
    for d in decls:
        if d.name in seen:
            if seen[d.name].shape != d.shape:
                raise ModelError(f"tensor '{d.name}' is declared with shapes {seen[d.name].shape} and {d.shape}")
            continue
        seen[d.name] = d
        out.append(d)
    return out


def _check_category(category: str):
    if category not in ("mixer", "feed_forward"):
        raise ModelError(f"a sub-layer is a 'mixer' or a 'feed_forward', got category '{category}'")


def _mixers(spec: ModelSpec, layer: int):
    """The mixer descriptions of a layer with their classes.  Every mixer of a layer gets the schedule entry's one
    cache id, so at most one of them may keep a cache or a state."""
    out = [(m, part_class("mixer", m)) for m in spec.layers[layer].parts_of("mixer")]
    keepers = [m for m, cls in out if cls.cache_need(m) is not None or cls.state_need(m) is not None]
    if len(keepers) > 1:
        raise ModelError(f"layer {layer} has {len(keepers)} mixers that keep a cache or a state; a schedule entry "
                         f"names one cache, so a layer can have one such mixer")
    return out


def check_schedule(spec: ModelSpec):
    """The schedule names existing layers; every cache has exactly one writer, which runs before its readers."""
    if not spec.schedule:
        raise ModelError("the schedule is empty")
    writers: Dict[int, int] = {}
    for i, e in enumerate(spec.schedule):
        if not 0 <= e.layer < len(spec.layers):
            raise ModelError(f"schedule entry {i} names layer {e.layer}; the model has {len(spec.layers)}")
        for mixer, cls in _mixers(spec, e.layer):
            if cls.cache_need(mixer) is None and cls.state_need(mixer) is None:
                continue
            writes = cls.writes_cache(mixer) if hasattr(cls, "writes_cache") else True
            if writes:
                if e.cache in writers:
                    raise ModelError(f"cache {e.cache} is written by schedule entries {writers[e.cache]} and {i}")
                writers[e.cache] = i
            elif e.cache not in writers:
                raise ModelError(f"schedule entry {i} reads cache {e.cache} before any entry has written it")


def cache_needs(spec: ModelSpec):
    """(paged needs, fixed-size state needs) per cache id, asked of the mixers in the schedule."""
    check_schedule(spec)
    kv: Dict[int, KVNeed] = {}
    states: Dict[int, StateNeed] = {}
    for e in spec.schedule:
        for mixer, cls in _mixers(spec, e.layer):
            need = cls.cache_need(mixer)
            if need is not None:
                if e.cache in kv and kv[e.cache] != need:
                    raise ModelError(f"cache {e.cache} is used with different needs: {kv[e.cache]} and {need}")
                kv[e.cache] = need
            st = cls.state_need(mixer)
            if st is not None:
                if e.cache in states and states[e.cache] != st:
                    raise ModelError(f"state {e.cache} is used with different needs")
                states[e.cache] = st
    return kv, states


def _layer_tensor_names(layer) -> List[str]:
    names = []
    for sub in layer.sublayers:
        for kind, d in (("norm", sub.norm), (sub.category, sub.part), ("norm", sub.post_norm)):
            if d is not None:
                names += [t.name for t in part_class(kind, d).declare(d)]
    return names


class Model:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], rt: Runtime, consume: bool = False):
        """``consume``: a layer's tensors are taken out of ``weights`` as soon as its parts are built (unless a later
        layer names them too), so that tensors which a part has fused into a new one are given back layer by layer
        instead of standing twice in memory until the whole model is built."""
        check_schedule(spec)
        self.spec = spec
        self.rt = rt
        self.embedding = weights[spec.embedding]
        self.blocks = []
        last_use = {}
        if consume:
            for i, layer in enumerate(spec.layers):
                for name in _layer_tensor_names(layer):
                    last_use[name] = i
        for i, layer in enumerate(spec.layers):
            built = []
            for sub in layer.sublayers:
                _check_category(sub.category)
                # "no norm" is a part too: it is where the sub-layer before is added to the residual stream
                norm = part_class("norm", sub.norm)(sub.norm, weights, rt) if sub.norm is not None \
                    else NoNorm(None, weights, rt)
                post = part_class("norm", sub.post_norm)(sub.post_norm, weights, rt) \
                    if sub.post_norm is not None else None
                built.append(BuiltSubLayer(sub.category, part_class(sub.category, sub.part)(sub.part, weights, rt),
                                           norm, post))
            self.blocks.append(part_class("arrangement", _Arrangement(layer.arrangement))(layer, built))
            if consume:
                for name in _layer_tensor_names(layer):
                    if last_use[name] == i and name not in (spec.embedding, spec.lm_head):
                        weights.pop(name, None)
        self._takes_after = ["after" in inspect.signature(b.forward).parameters for b in self.blocks]
        self.final_norm = part_class("norm", spec.final_norm)(spec.final_norm, weights, rt)
        head = weights.get(spec.lm_head)
        if head is None:
            if not spec.lm_head_optional:
                raise ModelError(f"tensor '{spec.lm_head}' is missing and the model does not tie its head")
            head = self.embedding  # the table stands in (qwen3.rs:366-373)
        self.tied = head is self.embedding
        self.head = Linear(head, rt)

    def forward(self, ctx) -> torch.Tensor:
        """Run the step's rows through all scheduled layers; float32 logits [wanted rows, vocab]."""
        n = ctx.token_ids.shape[0]
        residual = torch.empty((n, self.spec.width), dtype=torch.float32, device=self.rt.device)
        kernels.embedding_gather(self.embedding, ctx.token_ids, residual, self.rt.dtype,
                                 1.0 if self.spec.embedding_scale is None else self.spec.embedding_scale)
        pending = None
        schedule = self.spec.schedule
        for k, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            # a block that wants to know what runs after it (to fold the norm between into the products around it)
            # is told; the last block's output goes to the last norm, which reads a choice of rows
            if k + 1 < len(schedule) and self._takes_after[entry.layer]:
                after = getattr(self.blocks[schedule[k + 1].layer], "entry", None)
                pending = block.forward(ctx, entry.cache, residual, pending, after=after() if after else None)
            else:
                pending = block.forward(ctx, entry.cache, residual, pending)
        if ctx.logit_rows.shape[0] == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.rt.device)
        h = self.final_norm.add_norm(residual, pending, rows=ctx.logit_rows)
        logits = self.head(h, out_dtype=torch.float32)
        if self.spec.logit_scale is not None or self.spec.logit_softcap is not None:
            kernels.logit_scale_softcap(logits, 1.0 if self.spec.logit_scale is None else self.spec.logit_scale,
                                        self.spec.logit_softcap, self.rt.dtype)
        return logits


class _Arrangement:
    """The arrangement's name as a description with a ``kind``."""

    def __init__(self, kind: str):
        self.kind = kind

"""Descriptions of a model as data: which parts, of which sizes, in which order.

An architecture turns its typed configuration into one :class:`ModelSpec`.
Nothing below names an architecture: every size and constant is a field, every
layer has its own list of sub-layers (a mixer or a feed-forward with its norms each), and the order in which
layers run is the ``schedule`` list, which may name a layer twice or let two
entries use one cache.

A part's description is any frozen dataclass with a ``kind`` string; the
``kind`` selects the implementation in :mod:`inferrs_b200.parts.registry`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One tensor that a part expects in the weight files.

    ``init`` tells the random-weights mode how to fill it: ``"normal"`` is
    N(0, 0.02), ``"norm"`` is 1 + U(-0.1, 0.1).  ``optional`` tensors may be
    absent; the part says what it does then.
    """

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    weight: str
    kind: str = "rms"


@dataclass(frozen=True)
class PositionSpec:
    """Rotation of the first ``rot_dim`` elements of each head by position.

    ``kind="rotary_split_half"`` pairs element ``i`` with ``i + rot_dim/2``;
    ``kind="rotary_interleaved"`` pairs element ``2i`` with ``2i + 1``;
    ``kind="none"`` leaves heads as they are.
    """

    kind: str = "rotary_split_half"
    rot_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache of keys and values.

    ``window``: a query at position i sees keys j with i - window < j <= i;
    ``None`` means all keys j <= i.  ``own_kv=False`` describes a layer that
    has no key/value projections and reads the cache that another schedule
    entry writes.
    """

    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float
    position: PositionSpec
    q_proj: str
    o_proj: str
    k_proj: Optional[str] = None
    v_proj: Optional[str] = None
    q_norm: Optional[NormSpec] = None
    k_norm: Optional[NormSpec] = None
    window: Optional[int] = None
    own_kv: bool = True
    kind: str = "attention"


@dataclass(frozen=True)
class GatedDenseSpec:
    """down( act(gate(x)) * up(x) )."""

    width: int
    inner: int
    gate_proj: str
    up_proj: str
    down_proj: str
    activation: str = "silu"
    kind: str = "gated_dense"


@dataclass(frozen=True)
class SubLayerSpec:
    """One sub-layer of a block: a part with what stands before and after it.

    ``category`` says which registry the part's ``kind`` is looked up in: ``"mixer"`` (it gets the
    layer's cache) or ``"feed_forward"``.  ``norm`` is applied to the residual stream before the part
    (``None``: the part reads the stream as it is); ``post_norm`` to the part's output before it is
    added to the stream (``None``: it is added as it is).
    """

    part: Any
    category: str
    norm: Optional[Any] = None
    post_norm: Optional[Any] = None


@dataclass(frozen=True)
class LayerSpec:
    """One block: its sub-layers, in order, and how they are arranged around the residual stream.

    ``arrangement="sequential"``: for every sub-layer in turn, x += post_norm(part(norm(x))).  A
    pre-norm block of a mixer and a feed-forward is two sub-layers with a ``norm`` each
    (:func:`pre_norm_layer`); a block with four norms gives both a ``post_norm`` too; a block of a
    mixer alone has one sub-layer.
    """

    sublayers: Tuple[SubLayerSpec, ...]
    arrangement: str = "sequential"

    def parts_of(self, category: str) -> Tuple[Any, ...]:
        return tuple(s.part for s in self.sublayers if s.category == category)

    @property
    def mixer(self) -> Any:
        """The layer's mixer description (the first, if it has several; None if it has none)."""
        return next(iter(self.parts_of("mixer")), None)

    @property
    def ffn(self) -> Any:
        """The layer's feed-forward description (the first, if it has several; None if it has none)."""
        return next(iter(self.parts_of("feed_forward")), None)

    def with_part(self, category: str, part: Any, index: int = 0) -> "LayerSpec":
        """A copy in which the ``index``-th sub-layer of ``category`` has another part."""
        seen, subs = 0, []
        for s in self.sublayers:
            if s.category == category:
                if seen == index:
                    s = SubLayerSpec(part=part, category=category, norm=s.norm, post_norm=s.post_norm)
                seen += 1
            subs.append(s)
        if seen <= index:
            raise ValueError(f"the layer has {seen} sub-layers of category '{category}', none with index {index}")
        return LayerSpec(sublayers=tuple(subs), arrangement=self.arrangement)


def pre_norm_layer(mixer_norm: Any, mixer: Any, ffn_norm: Any, ffn: Any) -> LayerSpec:
    """x += mixer(norm(x)); x += feed_forward(norm(x))."""
    return LayerSpec(sublayers=(SubLayerSpec(part=mixer, category="mixer", norm=mixer_norm),
                                SubLayerSpec(part=ffn, category="feed_forward", norm=ffn_norm)))


@dataclass(frozen=True)
class ScheduleEntry:
    """Run layer ``layer`` with cache ``cache``.

    ``cache`` numbers the caches (and fixed-size states) of the model.  Two
    entries with the same ``layer`` share weights; two entries with the same
    ``cache`` share keys and values (exactly one of them writes).
    """

    layer: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    width: int
    embedding: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    lm_head: str
    # True: the head tensor may be absent, the embedding table is used then.
    lm_head_optional: bool
    max_positions: int
    # embedding rows are multiplied by this as they are gathered (None: not at all)
    embedding_scale: Optional[float] = None
    # logits are multiplied by logit_scale and then squashed to cap * tanh(x / cap) (None: neither)
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = ""
    extra: Tuple[Tuple[str, Any], ...] = field(default_factory=tuple)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Every layer once, in order, each with a cache of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))

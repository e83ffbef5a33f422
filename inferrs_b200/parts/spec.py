"""Descriptions of a model as data: which parts, of which sizes, in which order.

An architecture turns its typed configuration into one :class:`ModelSpec`.
Nothing below names an architecture: every size and constant is a field, every
layer has its own mixer and feed-forward description, and the order in which
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
class LayerSpec:
    """One block: two sub-layers, each with its norm, and how they are arranged.

    ``arrangement="pre_norm"``: x += mixer(norm(x)); x += feed_forward(norm(x)).
    """

    mixer_norm: Any
    mixer: Any
    ffn_norm: Any
    ffn: Any
    arrangement: str = "pre_norm"


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
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = ""
    extra: Tuple[Tuple[str, Any], ...] = field(default_factory=tuple)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Every layer once, in order, each with a cache of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))

"""From a part description's ``kind`` to the class that runs it.

Five kinds of part can be registered: mixers, feed-forwards, norms, position
encodings and block arrangements.  A model is built by looking up the class of
every description in its :class:`~inferrs_b200.parts.spec.ModelSpec`; a test or
a user adds a part with one ``register_*`` call and a description dataclass of
their own, without touching this package.

Interfaces (``rt`` is a :class:`~inferrs_b200.runtime.Runtime`, ``weights`` a
dict from tensor name to tensor on the device):

mixer
    ``declare(spec) -> [TensorDecl]`` (static), ``cache_need(spec) -> KVNeed | None`` (static),
    ``state_need(spec) -> StateNeed | None`` (static), ``__init__(spec, weights, rt)``,
    ``forward(ctx, cache_id, h) -> y`` with h, y ``[rows, width]`` in the activation dtype.
feed-forward
    ``declare(spec)``, ``__init__(spec, weights, rt)``, ``forward(ctx, h) -> y``.
norm
    ``declare(spec)``, ``__init__(spec, weights, rt)``,
    ``add_norm(residual, delta, rows=None) -> h``: adds ``delta`` (or nothing) into the float32
    residual in place and returns the normalised rows in the activation dtype; with ``rows``
    it reads only those rows and writes nothing back.  ``norm(x) -> y``: the norm alone on rows in
    the activation dtype (used where a description puts a norm on a sub-layer's output).
position encoding
    ``__init__(spec, rt)``, ``tables() -> (cos, sin, rot_dim)``: float32 ``[max_positions, rot_dim/2]``
    tables that the rotation kernel indexes by position (``rot_dim`` 0: no rotation).  Optional attribute
    ``interleaved = True``: element ``2i`` of a head turns with ``2i + 1`` instead of ``i`` with ``i + rot_dim/2``.
arrangement
    ``__init__(spec, sublayers)`` with ``spec`` the layer's :class:`~inferrs_b200.parts.spec.LayerSpec` and
    ``sublayers`` its built sub-layers in order (:class:`~inferrs_b200.parts.blocks.BuiltSubLayer`: ``category``,
    ``part``, ``norm``, ``post_norm``; ``run(ctx, cache_id, h)`` calls the part the way its category wants),
    ``forward(ctx, cache_id, residual, pending) -> pending`` (``residual`` float32 ``[rows, width]``, updated in
    place; ``pending`` is a sub-layer output that has not been added yet, or None), and
    ``parts() -> iterable`` of every part object the block holds.  Optional: ``entry() -> BuiltSubLayer`` (the
    sub-layer that takes what the block before hands on) and a keyword ``after`` of ``forward`` (the next block's
    entry): with them a block may fold the norm between two products into those products.

Optional for mixers and feed-forwards: ``takes_scaled_rows(n_rows)`` / ``feeds_sink(n_rows)`` and a ``sink`` keyword
of ``forward``.  A part that has them may be handed :class:`~inferrs_b200.kernels.ScaledRows` in place of its norm's
output, and a :class:`~inferrs_b200.kernels.ResidualSink` in place of returning its result (see
:class:`~inferrs_b200.parts.blocks.SequentialBlock`); a part without them never sees either.

Every part may set ``graph_safe = True`` to say that its launches depend only on shapes and device
memory, never on host-side values of the step; a model whose parts all say so has its steps captured
into CUDA graphs.  A part without the attribute keeps the model's steps launched one by one.
"""
from __future__ import annotations

from typing import Any, Dict

_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "arrangement")
_REGISTRY: Dict[str, Dict[str, type]] = {c: {} for c in _CATEGORIES}


class PartError(ValueError):
    pass


def register_part(category: str, kind: str, cls: type, replace: bool = False) -> type:
    if category not in _REGISTRY:
        raise PartError(f"unknown part category '{category}'; one of {_CATEGORIES}")
    if kind in _REGISTRY[category] and not replace and _REGISTRY[category][kind] is not cls:
        raise PartError(f"{category} '{kind}' is already registered")
    _REGISTRY[category][kind] = cls
    return cls


def register_mixer(kind: str, cls: type, replace: bool = False) -> type:
    return register_part("mixer", kind, cls, replace)


def register_feed_forward(kind: str, cls: type, replace: bool = False) -> type:
    return register_part("feed_forward", kind, cls, replace)


def register_norm(kind: str, cls: type, replace: bool = False) -> type:
    return register_part("norm", kind, cls, replace)


def register_position(kind: str, cls: type, replace: bool = False) -> type:
    return register_part("position", kind, cls, replace)


def register_arrangement(kind: str, cls: type, replace: bool = False) -> type:
    return register_part("arrangement", kind, cls, replace)


def part_class(category: str, spec: Any) -> type:
    kind = getattr(spec, "kind", None)
    if kind is None:
        raise PartError(f"a {category} description needs a 'kind', got {spec!r}")
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise PartError(f"no {category} of kind '{kind}' is registered; known: {sorted(_REGISTRY[category])}") from None

"""Reading config.json and the registry from architecture name to model.

The reference reads config.json into a struct whose fields are all optional
(inferrs-models/src/config.rs:277-329), detects the architecture from
``architectures[]`` and then ``model_type`` (config.rs:342-387) and builds a
typed per-architecture configuration from it (config.rs:468-502).  Here the
same three steps are: :class:`RawConfig`, :func:`resolve_architecture` and the
``from_raw`` constructor of the architecture's typed configuration.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


class RawConfig:
    """config.json as it stands on disk: a dictionary with typed getters.

    Every getter names the key it reads, so that a wrong type is reported with
    the key and the value that was found.
    """

    def __init__(self, values: Dict[str, Any], source: str = "<dict>"):
        if not isinstance(values, dict):
            raise ConfigError(f"{source}: config must be a JSON object, got {type(values).__name__}")
        self.values = dict(values)
        self.source = source

    @classmethod
    def from_file(cls, path: str) -> "RawConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        if not os.path.isfile(path):
            raise ConfigError(f"no config.json at {path}")
        with open(path, "r", encoding="utf-8") as f:
            try:
                values = json.load(f)
            except json.JSONDecodeError as e:
                raise ConfigError(f"{path}: not valid JSON: {e}") from e
        return cls(values, source=path)

    def has(self, key: str) -> bool:
        return key in self.values and self.values[key] is not None

    def _get(self, key: str, default, kind, kind_name: str):
        if not self.has(key):
            return default
        v = self.values[key]
        if kind is float and isinstance(v, int) and not isinstance(v, bool):
            v = float(v)
        if isinstance(v, bool) and kind is not bool:
            raise ConfigError(f"{self.source}: key '{key}' must be {kind_name}, got {v!r}")
        if not isinstance(v, kind):
            raise ConfigError(f"{self.source}: key '{key}' must be {kind_name}, got {v!r}")
        return v

    def get_int(self, key: str, default: Optional[int] = None) -> Optional[int]:
        return self._get(key, default, int, "an integer")

    def get_float(self, key: str, default: Optional[float] = None) -> Optional[float]:
        return self._get(key, default, float, "a number")

    def get_bool(self, key: str, default: Optional[bool] = None) -> Optional[bool]:
        return self._get(key, default, bool, "true or false")

    def get_str(self, key: str, default: Optional[str] = None) -> Optional[str]:
        return self._get(key, default, str, "a string")

    def get_list(self, key: str, default: Optional[list] = None) -> Optional[list]:
        return self._get(key, default, list, "a list")


@dataclass(frozen=True)
class Architecture:
    """One entry of the registry.

    name        the string found in config.json's ``architectures``
    model_type  the ``model_type`` that selects it when ``architectures`` is absent
    config_cls  typed configuration with ``from_raw(RawConfig)``
    build_spec  typed configuration -> ``parts.spec.ModelSpec``
    """

    name: str
    model_type: Optional[str]
    config_cls: type
    build_spec: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable, model_type: Optional[str] = None,
                          replace: bool = False) -> Architecture:
    """Add an architecture.  ``name`` is matched exactly against config.json."""
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    arch = Architecture(name=name, model_type=model_type, config_cls=config_cls, build_spec=build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def registered_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: RawConfig) -> Architecture:
    """The registry entry that config.json names.

    ``architectures[]`` is looked at first, then ``model_type``
    (config.rs:342-387 has this order).  The reference matches substrings; an
    exact match is asked for here, so that a new architecture whose name
    contains an old one is refused instead of being run as the old one.
    """
    names = raw.get_list("architectures", []) or []
    for n in names:
        if isinstance(n, str) and n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = raw.get_str("model_type")
    if mt is not None:
        for arch in _ARCHITECTURES.values():
            if arch.model_type == mt:
                return arch
    raise ConfigError(
        f"{raw.source}: unsupported model architecture (architectures={names!r}, model_type={mt!r}); "
        f"registered: {registered_architectures()}"
    )


def generation_eos_ids(model_dir: str, vocab_size: int) -> Tuple[int, ...]:
    """The ``eos_token_id`` (one id or a list) of ``generation_config.json`` in a model folder; () if there is no such
    file or no such key.  Checkpoints name there the ids that end a turn beside config.json's own end-of-text id.  (The
    reference takes its stop ids from the tokenizer's files, inferrs/src/tokenizer.rs:329-353; this engine reads no
    tokenizer, so the two JSON files and the request's own list are where stop ids come from.)"""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return ()
    with open(path, "r", encoding="utf-8") as f:
        try:
            values = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    v = values.get("eos_token_id") if isinstance(values, dict) else None
    if v is None:
        return ()
    ids = [v] if isinstance(v, int) and not isinstance(v, bool) else v
    if not isinstance(ids, list) or any(isinstance(t, bool) or not isinstance(t, int) for t in ids):
        raise ConfigError(f"{path}: eos_token_id must be an integer or a list of integers, got {v!r}")
    for t in ids:
        if not 0 <= t < vocab_size:
            raise ConfigError(f"{path}: eos_token_id {t} is outside the vocabulary of {vocab_size}")
    return tuple(ids)


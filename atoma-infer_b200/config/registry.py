"""Registries: architecture name -> model builder, and part kind -> part class.

The reference picks its model at compile time (a cargo feature and a generic
parameter, server/src/main.rs:45, backends/src/lib.rs:10-13).  Here the name in
``config.json``'s ``architectures[0]`` (or, failing that, its ``model_type``) picks an ``Architecture`` at run time, and
each layer of the model spec an architecture returns names its parts by kind
("attention", "swiglu", "rmsnorm", "rope", "prenorm"; the model's two ends: "token", "linear"), which these
tables resolve.
Another architecture or another part is added by one ``register_*`` call from any
module; nothing in the engine names a model.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    """``parse_config(dict) -> config`` and ``build_spec(config) -> ModelSpec``."""

    name: str
    parse_config: Callable[[dict], Any]
    build_spec: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[str, Dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


_MODEL_TYPES: Dict[str, str] = {}  # config.json "model_type" -> architecture name, for folders without "architectures"


def register_architecture(name: str, parse_config, build_spec, *, replace: bool = False, model_type: str = "") -> None:
    """``model_type``: the value of config.json's ``model_type`` that also means this architecture (used only
    when the file has no ``architectures`` list)."""
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)
    if model_type:
        _MODEL_TYPES[model_type] = name


def architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"architecture {name!r} is not registered (known: {sorted(_ARCHITECTURES)})"
        ) from None


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_of(model_dir: str):
    """Reads ``config.json`` of a model folder; returns (Architecture, typed config)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir!r} holds no config.json")
    with open(path) as f:
        raw = json.load(f)
    archs = raw.get("architectures")
    if archs and isinstance(archs, list):
        name = str(archs[0])
    elif raw.get("model_type") in _MODEL_TYPES:
        name = _MODEL_TYPES[raw["model_type"]]
    else:
        raise ConfigError("config.json has no 'architectures' list and no known 'model_type' "
                          f"(known architectures: {sorted(_ARCHITECTURES)}; model types: {sorted(_MODEL_TYPES)})")
    arch = architecture(name)
    return arch, arch.parse_config(raw)


def register_part(family: str, kind: str, cls: type, *, replace: bool = False) -> None:
    """family: 'mixer' | 'feed_forward' | 'norm' | 'position' | 'block' | 'embedding' | 'head'."""
    if family not in _PARTS:
        raise ConfigError(f"unknown part family {family!r} (known: {sorted(_PARTS)})")
    if kind in _PARTS[family] and not replace:
        raise ConfigError(f"{family} kind {kind!r} is already registered")
    _PARTS[family][kind] = cls


def part_class(family: str, kind: str) -> type:
    try:
        return _PARTS[family][kind]
    except KeyError:
        raise ConfigError(
            f"{family} kind {kind!r} is not registered (known: {sorted(_PARTS.get(family, {}))})"
        ) from None

"""One registry from an architecture's name to its configuration class and model.

``config.json`` names its model class in ``architectures[0]``.  The reference has
no registry: its engine hard-wires the one model it knows (include/engine.h:15-19).
An architecture registers a configuration class and a function that turns a
configuration into a ``ModelSpec`` (toyinfer_b200.parts.model); everything else
(weights, cache, step function, generation) works from that description.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

from .base import ConfigError, ModelConfig, read_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    describe: Callable[[ModelConfig], Any]  # config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, describe: Callable) -> None:
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_cls, describe)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(registered_architectures()) or '(none)'}"
        ) from None


def architecture_of(raw: Dict[str, Any], source: str = "config") -> Architecture:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{source}: 'architectures' must be a non-empty list of strings")
    return resolve_architecture(archs[0])


def load_config(model_dir: str) -> Tuple[Architecture, ModelConfig]:
    """Read ``model_dir/config.json`` and build the typed configuration it names."""
    path = os.path.join(model_dir, "config.json")
    raw = read_json(path)
    arch = architecture_of(raw, path)
    return arch, arch.config_cls.from_dict(raw, source=path)

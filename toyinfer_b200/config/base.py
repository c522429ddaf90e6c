"""Typed model configuration read from a checkpoint's ``config.json``.

A configuration class lists its keys once, as ``Key`` descriptors: the JSON key,
the accepted type, whether it is required and its default.  ``ModelConfig.from_dict``
checks presence and type of every key in one pass and raises a single
``ConfigError`` that names all problems.  Nothing here knows a model size; every
number comes from the file.

The reference reads twelve keys with ``asInt()/asFloat()`` and no presence check
(src/config.cpp:26-37), so a missing key silently becomes 0 there; here it is an
error.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be used; the message lists every problem found."""


_MISSING = object()


@dataclass(frozen=True)
class Key:
    """One key of config.json.

    ``kind`` is one of ``int``, ``float``, ``bool``, ``str``, ``int_or_list``
    (an int or a list of ints, normalised to a tuple), ``str_list``, ``any``.
    ``default`` may be a callable taking the partially built dict of earlier keys.
    """

    kind: str
    required: bool = True
    default: Any = None
    nullable: bool = False
    doc: str = ""


def _check(kind: str, name: str, value: Any) -> Tuple[Any, Optional[str]]:
    if kind == "int":
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value), None
            return None, f"{name}: expected an integer, got {value!r}"
        return value, None
    if kind == "float":
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            return None, f"{name}: expected a number, got {value!r}"
        return float(value), None
    if kind == "bool":
        if not isinstance(value, bool):
            return None, f"{name}: expected true/false, got {value!r}"
        return value, None
    if kind == "str":
        if not isinstance(value, str):
            return None, f"{name}: expected a string, got {value!r}"
        return value, None
    if kind == "int_or_list":
        if isinstance(value, int) and not isinstance(value, bool):
            return (value,), None
        if isinstance(value, list) and all(
            isinstance(v, int) and not isinstance(v, bool) for v in value
        ):
            return tuple(value), None
        return None, f"{name}: expected an integer or a list of integers, got {value!r}"
    if kind == "str_list":
        if isinstance(value, list) and all(isinstance(v, str) for v in value):
            return tuple(value), None
        return None, f"{name}: expected a list of strings, got {value!r}"
    if kind == "any":
        return value, None
    raise AssertionError(f"unknown key kind {kind}")


class ModelConfig:
    """Base of all architecture configurations.

    Subclasses set ``KEYS`` (ordered mapping key name -> ``Key``) and may override
    ``validate`` to check relations between keys; ``validate`` returns a list of
    problem strings.  Every key becomes an attribute of the instance.
    """

    KEYS: Dict[str, Key] = {}

    def __init__(self, values: Dict[str, Any]):
        for k, v in values.items():
            setattr(self, k, v)
        self._values = dict(values)

    # -- construction -----------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any], source: str = "config") -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"{source}: top level must be a JSON object")
        problems: List[str] = []
        values: Dict[str, Any] = {}
        for name, key in cls.KEYS.items():
            value = raw.get(name, _MISSING)
            if value is _MISSING or (value is None and not key.nullable and not key.required):
                if key.required and value is _MISSING:
                    problems.append(f"{name}: missing")
                    continue
                default = key.default
                if callable(default):
                    try:
                        default = default(values)
                    except Exception as exc:  # a default that needs a missing key
                        problems.append(f"{name}: cannot derive default ({exc})")
                        continue
                values[name] = default
                continue
            if value is None:
                if key.nullable:
                    values[name] = None
                    continue
                problems.append(f"{name}: null is not allowed")
                continue
            checked, err = _check(key.kind, name, value)
            if err:
                problems.append(err)
            else:
                values[name] = checked
        if problems:
            raise ConfigError(f"{source}: " + "; ".join(problems))
        cfg = cls(values)
        problems = cfg.validate()
        if problems:
            raise ConfigError(f"{source}: " + "; ".join(problems))
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "ModelConfig":
        return cls.from_dict(read_json(path), source=path)

    def validate(self) -> List[str]:
        return []

    # -- output -----------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for k, v in self._values.items():
            out[k] = list(v) if isinstance(v, tuple) else v
        return out

    def __repr__(self) -> str:
        body = ", ".join(f"{k}={v!r}" for k, v in self._values.items())
        return f"{type(self).__name__}({body})"


def read_json(path: str) -> Dict[str, Any]:
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: file not found")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from exc

"""Typed configurations and the architecture registry."""
from .base import ConfigError, Key, ModelConfig, read_json
from .qwen3 import Qwen3Config
from .registry import (
    Architecture,
    architecture_of,
    load_config,
    register_architecture,
    registered_architectures,
    resolve_architecture,
    unregister_architecture,
)

__all__ = [
    "ConfigError",
    "Key",
    "ModelConfig",
    "read_json",
    "Qwen3Config",
    "Architecture",
    "architecture_of",
    "load_config",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]

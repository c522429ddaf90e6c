"""Architectures this library knows; importing the package registers them."""
from . import qwen3  # noqa: F401

"""Random weights from a configuration and a seed.

Matrices are drawn from N(0, 0.02) and norm weights from 1 + N(0, 0.02), each tensor
from a generator seeded by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist or on the order of drawing.  ``write_model_folder`` writes
``config.json`` and ``model.safetensors`` (bfloat16 unless told otherwise);
``random_parameters`` fills tensors on the device without a file, for measurements at
sizes whose file would be large.  The reference has no such mode.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict

import torch

from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def draw(spec: ParamSpec, name: str, seed: int, device="cpu") -> torch.Tensor:
    """float32 draw of one tensor (int32 for integer tables)."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.role == "int_table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=torch.float32, device=device)
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    t.normal_(0.0, spec.std, generator=g)
    if spec.init == "one_plus_normal":
        t += 1.0
    elif spec.init != "normal":
        raise ValueError(f"{name}: unknown init {spec.init!r}")
    return t


def write_model_folder(config: Dict[str, Any], seed: int, out_dir: str,
                       store_dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors`` for the
    architecture that ``config`` names; returns ``out_dir``."""
    from ..config.registry import architecture_of
    from ..parts.model import DecoderModel

    arch = architecture_of(config)
    cfg = arch.config_cls.from_dict(config)
    model = DecoderModel(arch.describe(cfg), torch.float32, "cpu")
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=1)

    def tensors():
        for name, spec in model.param_specs().items():
            t = draw(spec, name, seed)
            yield name, (t if t.dtype == torch.int32 else t.to(store_dtype))

    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors())
    return out_dir


def random_parameters(specs: Dict[str, ParamSpec], seed: int, dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """Draws every tensor on ``device`` in the engine's dtype (values differ from the
    CPU draws of ``write_model_folder``: the generators are not the same)."""
    out = {}
    for name, spec in specs.items():
        t = draw(spec, name, seed, device=device)
        out[name] = t if t.dtype == torch.int32 else t.to(dtype)
    return out

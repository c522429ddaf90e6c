"""Loading a model's tensors from safetensors, by name.

The model says which tensors it wants (``param_specs``: name -> shape and role); the
loader finds each by its name, checks its shape and dtype, and puts it on the device:
matrices and tables follow the engine's dtype (bfloat16 checkpoints are widened for a
32-bit engine), integer tables become int32, and a tensor stored in 32-bit is never
narrowed: a norm weight stays float32, a 32-bit matrix is refused by a bfloat16 engine.
All problems of a checkpoint (missing tensors, tensors nobody asked for, wrong shapes,
unusable dtypes) are reported in one ``WeightError``.

The reference instead addresses one fixed model's tensors through a table of byte
offsets compiled into the binary (src/qwen.cpp:17-416, :482-515), made offline by
export.py:211-320; a checkpoint of another size is silently misread there.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import SafetensorsError, open_model

_FLOATS = (torch.bfloat16, torch.float16, torch.float32)
_INTS = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)


class WeightError(ValueError):
    """A checkpoint that does not fit the model; lists every problem found."""


def _target_dtype(name: str, spec: ParamSpec, stored: torch.dtype, engine: torch.dtype) -> Tuple[torch.dtype, str]:
    """dtype to keep the tensor in, or an error string."""
    if spec.role == "int_table":
        if stored not in _INTS:
            return stored, f"{name}: an integer table is stored as {stored}"
        return torch.int32, ""
    if stored not in _FLOATS:
        return stored, f"{name}: stored as {stored}, expected a floating-point tensor"
    if engine == torch.float32:
        return torch.float32, ""
    # bfloat16 engine
    if stored == torch.float32:
        if spec.role == "norm":
            return torch.float32, ""
        return stored, (
            f"{name}: stored in float32; a bfloat16 engine does not narrow 32-bit tensors "
            "(run with dtype float32)"
        )
    return torch.bfloat16, ""


def load_parameters(
    specs: Dict[str, ParamSpec],
    model_dir: str,
    dtype: torch.dtype,
    device,
    ignorable: Iterable[str] = (),
) -> Dict[str, torch.Tensor]:
    try:
        files, where = open_model(model_dir)
    except SafetensorsError as exc:
        raise WeightError(str(exc)) from exc
    try:
        missing: List[str] = []
        wrong: List[str] = []
        for name, spec in specs.items():
            f = where.get(name)
            if f is None:
                missing.append(name)
                continue
            e = f.entries[name]
            if tuple(e.shape) != tuple(spec.shape):
                wrong.append(f"{name}: shape {list(e.shape)} in the file, {list(spec.shape)} expected")
                continue
            _, err = _target_dtype(name, spec, e.dtype, dtype)
            if err:
                wrong.append(err)
        ignorable = set(ignorable)
        unexpected = sorted(n for n in where if n not in specs and n not in ignorable)
        if missing or wrong or unexpected:
            lines = [f"{model_dir}: the checkpoint does not fit the model"]
            if missing:
                lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
            if unexpected:
                lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
            raise WeightError("\n".join(lines))
        out: Dict[str, torch.Tensor] = {}
        for name, spec in specs.items():
            f = where[name]
            tgt, _ = _target_dtype(name, spec, f.entries[name].dtype, dtype)
            cpu = f.tensor(name)
            # one shard-sized staging copy at a time: .to() of a mapped view streams it
            # always a copy: the mapped file is closed when loading ends
            out[name] = cpu.to(device=device, dtype=tgt, copy=True).contiguous()
        return out
    finally:
        for f in files:
            f.close()

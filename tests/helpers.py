"""Comparison rules shared by the model-level tests."""
from __future__ import annotations

import torch

from plain import qwen3_plain as plain


def rounding_of(dtype: str):
    return None if dtype == "float32" else torch.bfloat16


def assert_logits_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    """float32 engine: |got - want| <= 1e-5 + 1e-4 |want| against the exact (float64)
    plain result.  bfloat16 engine, against the plain result rounded at the same places:
    values that differ in summation order round differently now and then, one bfloat16
    step (2^-8) at a time, so the bound is 2 % of the row's largest logit plus 2 %."""
    got = got.detach().cpu().double()
    want = want.detach().cpu().double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5, msg=lambda m: f"{what}: {m}")
    else:
        scale = want.abs().amax(dim=-1, keepdim=True)
        bound = 0.02 * scale + 0.02 * want.abs()
        bad = (got - want).abs() > bound
        assert not bad.any(), f"{what}: {int(bad.sum())} logits off, worst {(got - want).abs().max():.4g} vs scale {scale.max():.4g}"


_cache = {}


def plain_logits(folder: str, ids, dtype: str) -> torch.Tensor:
    key = (folder, tuple(ids), dtype)
    if key not in _cache:
        if folder not in _cache:
            _cache[folder] = (plain.read_weights(folder), plain.read_config(folder))
        w, cfg = _cache[folder]
        _cache[key] = plain.forward(w, cfg, ids, rounding_of(dtype))
    return _cache[key]

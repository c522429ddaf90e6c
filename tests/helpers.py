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


def run_random_schedule(eng, ids, rng, max_live=4):
    """Feeds the requests ``ids`` (lists of tokens) through the engine as a random schedule decides:
    a step takes a random subset of the live sequences, each with a random number of its next
    tokens (one, a few, a long piece, all that is left); new sequences start beside them; a
    finished one gives its slot and pages back at once.  Returns, per request, the logits of all
    its positions in order."""
    import torch
    lens = [len(x) for x in ids]
    waiting = list(range(len(ids)))
    live = {}                    # request -> (slot, tokens fed)
    got = {r: [] for r in range(len(ids))}
    steps = 0
    while waiting or live:
        steps += 1
        assert steps < 5000, "the schedule does not end"
        while waiting and len(live) < max_live and (not live or rng.random() < 0.5):
            live[waiting.pop(0)] = (eng.new_sequence(), 0)
        chosen = [r for r in live if rng.random() < 0.7] or [rng.choice(list(live))]
        entries, wants = [], []
        for r in chosen:
            slot, fed = live[r]
            left = lens[r] - fed
            take = min(left, rng.choice([1, 1, 1, 2, 5, 64, 70, left]))
            entries.append((slot, ids[r][fed:fed + take]))
            wants.append(list(range(take)))
            live[r] = (slot, fed + take)
        out = eng.step(entries, wants).clone()
        o = 0
        for r, w in zip(chosen, wants):
            got[r].append(out[o:o + len(w)])
            o += len(w)
        for r in chosen:
            slot, fed = live[r]
            assert eng.length(slot) == fed
            if fed == lens[r]:
                eng.end_sequence(slot)
                del live[r]
    return [torch.cat(got[r]) for r in range(len(ids))]

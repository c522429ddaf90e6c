"""The plain implementation's parts against the reference's own CPU oracles
(tests/golden/reference_ops.json, made by tests/golden/make_golden.py)."""
from __future__ import annotations

import json
import math
import os

import pytest
import torch

from plain import qwen3_plain as plain

HERE = os.path.dirname(os.path.abspath(__file__))
BF16 = dict(rtol=8e-3, atol=1e-6)      # both sides round to bfloat16: one step apart at most


@pytest.fixture(scope="module")
def gold():
    with open(os.path.join(HERE, "golden", "reference_ops.json")) as f:
        return json.load(f)


def t(x):
    return torch.tensor(x, dtype=torch.float64)


def test_rmsnorm(gold):
    g = gold["rmsnorm"]
    got = plain.rms_norm(t(g["x"])[None], t(g["w"]), g["eps"], torch.bfloat16)[0]
    torch.testing.assert_close(got, t(g["y"]), **BF16)


def test_head_rmsnorm(gold):
    g = gold["head_rmsnorm"]
    x = t(g["x"]).view(1, g["heads"], g["head_dim"])
    got = plain.rms_norm(x, t(g["w"]), g["eps"], torch.bfloat16).reshape(-1)
    torch.testing.assert_close(got, t(g["y"]), **BF16)


def test_rope_pairs_and_signs(gold):
    g = gold["rope"]
    x = t(g["x"]).view(1, g["heads"], g["head_dim"])
    ang = (torch.tensor(g["inv_freq"], dtype=torch.float32) * float(g["pos"])).double()[None]
    got = plain.rope(x, ang, torch.bfloat16).reshape(-1)
    torch.testing.assert_close(got, t(g["y"]), **BF16)


def test_inv_freq(gold):
    g = gold["inv_freq"]
    got = plain.rope_angles(g["head_dim"], g["theta"], [1])[0]
    torch.testing.assert_close(got, t(g["y"]), rtol=2e-6, atol=0)


def test_swiglu(gold):
    g = gold["swiglu"]
    got = plain.swiglu(t(g["gate"]), t(g["up"]), torch.bfloat16)
    torch.testing.assert_close(got, t(g["y"]), **BF16)


def test_causal_grouped_attention(gold):
    g = gold["attention"]
    T, nh, nkv, hd = g["seq"], g["heads"], g["kv_heads"], g["head_dim"]
    q, k, v = t(g["q"]).view(T, nh, hd), t(g["k"]).view(T, nkv, hd), t(g["v"]).view(T, nkv, hd)
    got = plain.attention(q, k, v, 1.0 / math.sqrt(hd)).reshape(-1)
    torch.testing.assert_close(got, t(g["y"]), rtol=1e-5, atol=1e-6)

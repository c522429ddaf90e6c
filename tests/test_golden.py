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


def test_linear_weight_layout(gold):
    """Weights are [out, in] row-major: 5 rows of 12, not square, so a transposed reading
    cannot pass (gemv_test::reference_sum)."""
    g = gold["gemv"]
    w = t(g["w"]).view(g["rows"], g["cols"])
    got = plain.linear(t(g["x"])[None], w)[0]
    torch.testing.assert_close(got, t(g["y"]), rtol=1e-5, atol=1e-6)


def test_decode_attention_scores_softmax_and_values(gold):
    """The reference's three decode-attention oracles (attention_test::reference_qk_scores,
    reference_softmax, reference_apply_score) against the last row of the plain attention: the
    query at position ``pos`` over the cache rows 0..pos, rows beyond it never read."""
    g = gold["decode_attention"]
    nh, nkv, hd, pos, rows = g["heads"], g["kv_heads"], g["head_dim"], g["pos"], g["rows"]
    T = pos + 1
    k = t(g["k"]).view(rows, nkv, hd)[:T]
    v = t(g["v"]).view(rows, nkv, hd)[:T]
    q = torch.zeros(T, nh, hd, dtype=torch.float64)
    q[-1] = t(g["q"]).view(nh, hd)
    scale = 1.0 / math.sqrt(hd)
    got = plain.attention(q, k, v, scale)[-1].reshape(-1)
    torch.testing.assert_close(got, t(g["o"]), rtol=1e-5, atol=1e-6)
    # the intermediate oracles, restated with the same elementary steps as plain.attention
    grp = nh // nkv
    scores = torch.stack([(k[:, h // grp, :] @ q[-1, h]) * scale for h in range(nh)])
    torch.testing.assert_close(scores, t(g["scores"]).view(nh, rows)[:, :T], rtol=1e-5, atol=1e-6)
    probs = torch.exp(scores - scores.max(dim=-1, keepdim=True).values)
    probs = probs / probs.sum(dim=-1, keepdim=True)
    torch.testing.assert_close(probs, t(g["probs"]).view(nh, rows)[:, :T], rtol=1e-5, atol=1e-6)
    assert torch.all(t(g["probs"]).view(nh, rows)[:, T:] == 0)


def test_residual_sum_rounds_once(gold):
    g = gold["residual_add"]
    got = plain.rnd(t(g["hidden"]) + t(g["residual"]), torch.bfloat16)
    # the same bfloat16 values; the file prints 9 significant digits
    torch.testing.assert_close(got, t(g["y"]), rtol=1e-7, atol=0)

"""Plain, slow Qwen3 dense: whole sequences, no cache, one function per part.

This file is the oracle of the tests.  It shares no code with toyinfer_b200: it reads
config.json as a dict, reads safetensors with its own few lines, and computes every
part with elementary torch operations in float64, on the device its inputs live on (the
CPU in most tests; a GPU when weights of real layer sizes are handed in on one, where the
same operations run in seconds).  Each function cites the lines of the reference
(wiketool/ToyInfer) whose formula it restates.

The reference's model code is CUDA only (every op is a __global__ kernel) and its host
program needs third-party sources that are not in its tree, so it cannot run on a
machine without a GPU: the composition of the parts rests on the formulas, not on a
run of the reference.  The per-op CPU oracles that the reference ships with its kernel
tests do compile; tests/golden holds their outputs next to this file's (see
tests/golden/README.md).

``rounding`` selects where values are rounded, to mirror an engine's storage type:
``None`` keeps float64 everywhere (the exact answer a 32-bit engine must approach);
``torch.bfloat16`` rounds at every place where the reference stores a bfloat16 value
(after each projection, norm, rotation, activation and residual sum), so that a
bfloat16 engine can be compared tightly.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------
# files
# ---------------------------------------------------------------------------
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        return json.load(f)


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header with dtype/shape/data_offsets per
    tensor, raw data (export.py:211-230 and :272-277 scan the same layout)."""
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        buf = bytearray(raw[8 + n + b:8 + n + e])
        t = torch.frombuffer(buf, dtype=kinds[meta["dtype"]]) if e > b else torch.empty(0, dtype=kinds[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for n in sorted(os.listdir(model_dir)):
        if n.endswith(".safetensors"):
            out.update(read_safetensors(os.path.join(model_dir, n)))
    return out


# ---------------------------------------------------------------------------
# rounding
# ---------------------------------------------------------------------------
def rnd(x: torch.Tensor, rounding: Optional[torch.dtype]) -> torch.Tensor:
    if rounding is None:
        return x
    return x.to(torch.float32).to(rounding).to(F64)


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """h[t] = E[id_t], no scale (src/prefill.cu:17-21, src/transformer.cpp:641-644)."""
    return table[torch.tensor(list(ids), dtype=torch.long, device=table.device)].to(F64)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, rounding=None) -> torch.Tensor:
    """y = x * rsqrt(sum(x^2)/n + eps) * w over the last dimension; the weight multiplies
    as it is, without 1 + w (src/decode.cu:118-123, src/prefill.cu:90-93)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return rnd(x * torch.rsqrt(ms + eps) * w.to(F64), rounding)


def linear(x: torch.Tensor, w: torch.Tensor, rounding=None) -> torch.Tensor:
    """y[r] = sum_c W[r, c] x[c], weights [out, in], no bias (src/decode.cu:213-234)."""
    return rnd(x @ w.to(F64).T, rounding)


def rope_angles(head_dim: int, theta: float, positions: Sequence[int]) -> torch.Tensor:
    """angle[p, i] = p * theta^(-2i/head_dim), i < head_dim/2 (src/decode.cu:35-41, :313)."""
    i = torch.arange(head_dim // 2, dtype=F64)
    inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=F64), 2.0 * i / head_dim)
    return torch.tensor(list(positions), dtype=F64)[:, None] * inv_freq[None, :]


def rope(x: torch.Tensor, angles: torch.Tensor, rounding=None) -> torch.Tensor:
    """x: [T, heads, head_dim].  Pairs (i, i + head_dim/2): a' = a cos - b sin,
    b' = b cos + a sin (src/decode.cu:313-322, src/prefill.cu:185-208).  The cos and sin
    are rounded to float32 first, as every engine reads them from 32-bit tables."""
    half = x.shape[-1] // 2
    c = torch.cos(angles).to(torch.float32).to(F64)[:, None, :]
    s = torch.sin(angles).to(torch.float32).to(F64)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return rnd(torch.cat([a * c - b * s, b * c + a * s], dim=-1), rounding)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
              rounding=None) -> torch.Tensor:
    """q [T, heads, d], k and v [T, kv_heads, d] of one sequence whose positions are
    0..T-1.  Query head h reads kv head h // (heads / kv_heads) (src/decode.cu:420,
    src/prefill.cu:265); s = (q.k) * scale for keys at positions <= the query's
    (src/prefill.cu:316) and, with a window, > position - window; softmax with the
    maximum subtracted (src/decode.cu:488-531); o = sum p v (src/decode.cu:618-627)."""
    T, nh, d = q.shape
    g = nh // k.shape[1]
    out = torch.zeros(T, nh, d, dtype=F64, device=q.device)
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= pos[None, :] > pos[:, None] - window
    for h in range(nh):
        s = (q[:, h, :] @ k[:, h // g, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, h // g, :]
    return rnd(out, rounding)


def swiglu(gate: torch.Tensor, up: torch.Tensor, rounding=None) -> torch.Tensor:
    """z = up * gate / (1 + exp(-gate)) (src/decode.cu:756-762)."""
    return rnd(up * (gate / (1.0 + torch.exp(-gate))), rounding)


def layer_window(cfg: dict, layer: int) -> int:
    """Window of a layer from the configuration's own keys: ``layer_types`` when present,
    else ``use_sliding_window`` applies ``sliding_window`` to layers >= max_window_layers.
    (The reference reads none of these keys: all its layers see every key.)"""
    lt = cfg.get("layer_types")
    if lt is not None:
        return int(cfg["sliding_window"]) if lt[layer] == "sliding_attention" else 0
    if cfg.get("use_sliding_window", False) and layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return int(cfg["sliding_window"])
    return 0


def decoder_layer(h: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict, layer: int,
                  rounding=None) -> torch.Tensor:
    """Pre-norm block in the reference's order (src/transformer.cpp:513-618): input norm,
    q/k/v projections, per-head q and k norm (before the rotation, :535-542), rotation,
    attention, output projection, residual sum, post-attention norm, SwiGLU feed-forward,
    residual sum.  h: [T, hidden] of one sequence at positions 0..T-1."""
    p = f"model.layers.{layer}."
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg["rms_norm_eps"]
    T = h.shape[0]
    x = rms_norm(h, w[p + "input_layernorm.weight"], eps, rounding)
    q = linear(x, w[p + "self_attn.q_proj.weight"], rounding).view(T, nh, hd)
    k = linear(x, w[p + "self_attn.k_proj.weight"], rounding).view(T, nkv, hd)
    v = linear(x, w[p + "self_attn.v_proj.weight"], rounding).view(T, nkv, hd)
    q = rms_norm(q, w[p + "self_attn.q_norm.weight"], eps, rounding)
    k = rms_norm(k, w[p + "self_attn.k_norm.weight"], eps, rounding)
    ang = rope_angles(hd, cfg["rope_theta"], range(T)).to(h.device)
    q, k = rope(q, ang, rounding), rope(k, ang, rounding)
    a = attention(q, k, v, 1.0 / math.sqrt(hd), layer_window(cfg, layer), rounding)
    o = linear(a.reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"], rounding)
    h = rnd(h + o, rounding)                                   # src/decode.cu:18-19
    x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, rounding)
    gate = linear(x, w[p + "mlp.gate_proj.weight"], rounding)
    up = linear(x, w[p + "mlp.up_proj.weight"], rounding)
    m = linear(swiglu(gate, up, rounding), w[p + "mlp.down_proj.weight"], rounding)
    return rnd(h + m, rounding)


def forward(w: Dict[str, torch.Tensor], cfg: dict, ids: Sequence[int], rounding=None,
            rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of every position of one whole sequence (or of the
    positions in ``rows`` only): embedding, layers, final norm, head
    (src/transformer.cpp:345-470).  The head is the embedding table when
    ``tie_word_embeddings`` is true (the reference always ties, src/qwen.cpp:482-483) and
    ``lm_head.weight`` otherwise; its output is not rounded (float32 logits,
    src/decode.cu:251-286)."""
    h = rnd(embedding(w["model.embed_tokens.weight"], ids), rounding)
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, cfg, layer, rounding)
    if rows is not None:
        h = h[torch.tensor(list(rows), dtype=torch.long, device=h.device)]
    x = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"], rounding)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, head, None)


# ---------------------------------------------------------------------------
# choosing tokens
# ---------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> int:
    """First maximum wins (src/sampler.cpp:71-81)."""
    best, idx = -math.inf, 0
    for i, v in enumerate(logits.tolist()):
        if v > best:
            best, idx = v, i
    return idx


_M64 = (1 << 64) - 1


def uniform_from(seed: int, key: int, step: int) -> float:
    """The library's uniform number for (seed, sequence key, step): a 64-bit mix of the
    three, top 24 bits scaled to [0, 1).  (The reference draws from a clock-seeded
    mt19937, src/sampler.cpp:57-60, which cannot be reproduced.)"""
    x = (seed * 0x9E3779B97F4A7C15 + key * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & _M64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M64
    x ^= x >> 31
    return (x >> 40) / 16777216.0


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """The reference's order (src/sampler.cpp:24-68): x = logit / temperature; keep the
    top_k largest; p = softmax over them; sort descending; cut after the first entry at
    which the running sum exceeds top_p; coin = u * that sum; the first entry whose
    running sum exceeds the coin.  The temperature divides once (the reference divides
    again inside the exponent, :38).  Ties are ordered by lower index first.  Computed
    in float32 like the library, summing in list order."""
    x = (logits.to(torch.float32) / torch.tensor(temperature, dtype=torch.float32))
    V = x.numel()
    order = sorted(range(V), key=lambda i: (-x[i].item(), i))
    k = top_k if 0 < top_k < V else V
    kept = order[:k]
    if k == V and top_p >= 1.0:
        # no limits: the running sum goes over the vocabulary in index order
        m = x.max()
        p = torch.exp(x - m)
        total = torch.tensor(0.0, dtype=torch.float32)
        for v in p:
            total = total + v
        target = torch.tensor(u, dtype=torch.float32) * total
        acc = torch.tensor(0.0, dtype=torch.float32)
        for i in range(V):
            acc = acc + p[i]
            if acc > target:
                return i
        return V - 1
    vals = x[kept]
    p = torch.exp(vals - vals[0])
    s = torch.tensor(0.0, dtype=torch.float32)
    for v in p:
        s = s + v
    acc = torch.tensor(0.0, dtype=torch.float32)
    n = k
    for i in range(k):
        acc = acc + p[i] / s
        if acc > top_p:
            n = i + 1
            break
    coin = torch.tensor(u, dtype=torch.float32) * acc
    run = torch.tensor(0.0, dtype=torch.float32)
    for i in range(n):
        run = run + p[i] / s
        if run > coin:
            return kept[i]
    return kept[n - 1]


def generate(w, cfg, prompt: Sequence[int], max_new_tokens: int, stop_ids=(), temperature: float = 0.0,
             top_k: int = 1, top_p: float = 1.0, seed: int = 0, key: int = 0, rounding=None,
             max_seq_len: Optional[int] = None) -> List[int]:
    """Greedy or sampled continuation, recomputing the whole sequence for every token.
    Stop tokens end the sequence and are not part of the output
    (src/engine_runtime.cpp:448-450); so do max_new_tokens and max_seq_len (:459-463)."""
    ids = list(prompt)
    out: List[int] = []
    limit = max_seq_len or cfg["max_position_embeddings"]
    greedy = abs(temperature) < 1e-3 or top_k == 1            # src/sampler.cpp:20
    while len(out) < max_new_tokens and len(ids) < limit:
        logits = forward(w, cfg, ids, rounding)[-1]
        if greedy:
            tok = argmax(logits)
        else:
            tok = sample(logits, temperature, top_k, top_p, uniform_from(seed, key, len(out)))
        if tok in stop_ids:
            break
        out.append(tok)
        ids.append(tok)
    return out

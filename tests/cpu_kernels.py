"""Stand-ins for toyinfer_b200.kernels written with torch on the CPU, for tests only.

The library has no CPU path.  These functions let the tests that run without a GPU
drive the library's own engine, cache, batch metadata and generation loop (everything
around the kernels) by patching the kernel module's functions; they follow the same
calling conventions, including the paged cache layout, so that slot and page handling
is exercised for real.  ``install(monkeypatch)`` patches them in.
"""
from __future__ import annotations

import math

import torch

import toyinfer_b200.kernels as K


def embed(table, ids, scale=1.0):
    out = table[ids.long()].clone()
    return out if scale == 1.0 else (out.float() * scale).to(table.dtype)


def logit_scale_cap(logits, scale=1.0, cap=0.0):
    logits.mul_(scale)
    if cap > 0:
        logits.copy_(cap * torch.tanh(logits / cap))
    return logits


def rmsnorm(x, w, eps):
    xf = x.float()
    r = torch.rsqrt((xf * xf).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (xf * r * w.float()).to(x.dtype)


def add_rmsnorm(h, delta, w, eps):
    h.copy_((h.float() + delta.float()).to(h.dtype))
    return rmsnorm(h, w, eps)


def gather_add(h, delta, rows):
    out = h[rows.long()].float()
    if delta is not None:
        out = out + delta[rows.long()].float()
    return out.to(h.dtype)


def linear(x, w, out_dtype=None, late_start=False):
    if isinstance(x, K.PendingNorm):
        x = x.tensor()
    return (x.float() @ w.float().T).to(out_dtype or x.dtype)


def swiglu(gu, pairs=False):
    i = gu.shape[1] // 2
    g, u = (gu[:, 0::2].float(), gu[:, 1::2].float()) if pairs else (gu[:, :i].float(), gu[:, i:].float())
    return (u * (g / (1.0 + torch.exp(-g)))).to(gu.dtype)


def linear_swiglu(x, w_pairs):
    return swiglu(linear(x, w_pairs), pairs=True)


class PendingOutOfPlace(K.PendingNorm):
    """A pending norm whose sum lands in a new tensor, as after the product that forms its own
    input; h itself stays as it was."""

    def tensor(self):
        if self._x is None:
            summed = self.h if self.delta is None else (self.h.float() + self.delta.float()).to(self.h.dtype)
            self._hidden = summed.clone()
            self._x = rmsnorm(self._hidden, self.weight, self.eps)
        return self._x


def _norm_heads(x, w, eps):
    xf = x.float()
    r = torch.rsqrt((xf * xf).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (xf * r * w.float()).to(x.dtype)


def _rotate(x, cos, sin, pos):
    half = x.shape[-1] // 2
    c, s = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


def qk_norm_rope_store(q, k, v, q_w, k_w, eps, tables, batch, mem):
    if q is not None:
        if q_w is not None:
            q.copy_(_norm_heads(q, q_w, eps))
        if tables is not None:
            q.copy_(_rotate(q, tables[0], tables[1], batch.tok_pos))
    if k is not None:
        if k_w is not None:
            k.copy_(_norm_heads(k, k_w, eps))
        if tables is not None:
            k.copy_(_rotate(k, tables[0], tables[1], batch.tok_pos))
    if mem is not None:
        pos, seq = batch.tok_pos.tolist(), batch.tok_seq.tolist()
        slots, lens = batch.seq_slot.tolist(), batch.seq_len.tolist()
        for m in range(len(pos)):
            p, s = pos[m], seq[m]
            row = p
            if mem.ring_rows:
                if p < lens[s] - mem.ring_rows:
                    continue
                row = p % mem.ring_rows
            page = int(mem.page_table[slots[s], row // mem.page_size])
            line = row % mem.page_size
            if k is not None:
                mem.k_pages[page, :, line, :] = k[m]
            if v is not None:
                mem.v_pages[page, :, line, :] = v[m]


def _attend(q, k, v, scale, lo):
    """q [heads, d]; k, v [n, kv_heads, d] are the visible keys; returns [heads, d]."""
    nh, nkv = q.shape[0], k.shape[1]
    g = nh // nkv
    out = torch.zeros_like(q, dtype=torch.float32)
    for h in range(nh):
        s = (k[:, h // g, :].float() @ q[h].float()) * scale
        p = torch.softmax(s, dim=0)
        out[h] = p @ v[:, h // g, :].float()
    return out


def attention_prefill(q, k, v, scale, window, batch):
    out = torch.empty_like(q)
    cu = batch.cu_new.tolist()
    for b in range(batch.n_seq):
        t0, t1 = cu[b], cu[b + 1]
        for i in range(t1 - t0):
            lo = max(0, i - window + 1) if window > 0 else 0
            out[t0 + i] = _attend(q[t0 + i], k[t0 + lo:t0 + i + 1], v[t0 + lo:t0 + i + 1], scale, lo).to(q.dtype)
    return out


def attention_chunk(q, k, v, mem, scale, window, batch):
    out = torch.empty_like(q)
    cu, starts, slots = batch.cu_new.tolist(), batch.seq_start.tolist(), batch.seq_slot.tolist()
    for b in range(batch.n_seq):
        t0, t1, st = cu[b], cu[b + 1], starts[b]
        for i in range(t1 - t0):
            pos = st + i
            lo = max(0, pos - window + 1) if window > 0 else 0
            ks, vs = [], []
            for p in range(lo, pos + 1):
                if p >= st:
                    ks.append(k[t0 + p - st])
                    vs.append(v[t0 + p - st])
                else:
                    row = p % mem.ring_rows if mem.ring_rows else p
                    page = int(mem.page_table[slots[b], row // mem.page_size])
                    ks.append(mem.k_pages[page, :, row % mem.page_size, :])
                    vs.append(mem.v_pages[page, :, row % mem.page_size, :])
            out[t0 + i] = _attend(q[t0 + i], torch.stack(ks), torch.stack(vs), scale, lo).to(q.dtype)
    return out


def attention_decode(q, mem, scale, window, batch):
    out = torch.empty_like(q)
    slots, lens = batch.seq_slot.tolist(), batch.seq_len.tolist()
    for b in range(q.shape[0]):
        L = lens[b]
        lo = max(0, L - window) if window > 0 else 0
        ks, vs = [], []
        for p in range(lo, L):
            row = p % mem.ring_rows if mem.ring_rows else p
            page = int(mem.page_table[slots[b], row // mem.page_size])
            ks.append(mem.k_pages[page, :, row % mem.page_size, :])
            vs.append(mem.v_pages[page, :, row % mem.page_size, :])
        out[b] = _attend(q[b], torch.stack(ks), torch.stack(vs), scale, lo).to(q.dtype)
    return out


def attention_decode_step(q, k, v, q_w, k_w, eps, tables, mem, scale, window, batch):
    qk_norm_rope_store(q, k, v, q_w, k_w, eps, tables, batch, mem if k is not None else None)
    return attention_decode(q, mem, scale, window, batch)


def argmax(logits):
    return torch.argmax(logits, dim=1).to(torch.int32)


def install(monkeypatch) -> None:
    for name in ("embed", "logit_scale_cap", "rmsnorm", "add_rmsnorm", "gather_add", "linear", "swiglu", "linear_swiglu", "qk_norm_rope_store",
                 "attention_prefill", "attention_chunk", "attention_decode", "attention_decode_step", "argmax"):
        monkeypatch.setattr(K, name, globals()[name])

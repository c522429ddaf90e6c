"""Grouped-query attention mixer.

For each token x: q = Wq x, k = Wk x, v = Wv x (no bias; weights [out, in],
src/decode.cu:202-236, src/transformer.cpp:521-533); optional per-head RMS norm of
q and k over head_dim with one weight shared by all heads, before the rotation
(src/decode.cu:144-187, src/transformer.cpp:535-542); position encoding of q and k
(parts/rope.py); k and v are stored in the cache at the token's position
(src/transformer.cpp:549-552); query head h reads kv head h // (heads / kv_heads)
(src/decode.cu:420); scores (q.k) * head_dim^-0.5 over the keys at positions
<= the query's (and > position - window when the layer has a window), softmax in
32-bit, weighted sum of v (src/decode.cu:401-432, :471-532, :598-628;
src/prefill.cu:224-379); then o = Wo a (src/transformer.cpp:574-577).

Parameters choose everything: head counts, head size, norm on or off and its eps,
the window, the name of the position encoding, whether the layer has keys and
values of its own (``own_kv``) or reads those of the entry it borrows memory from,
and the softmax scale.

A step may continue each sequence from any position by any number of tokens
(``batch.mode == "mixed"``): a token's keys are then the sequence's earlier positions,
read from the cache, and the step's own tokens up to itself.  Two special cases have
kernels of their own: every sequence starts at position 0 (``"start"``: all keys are the
step's own) and every sequence goes on by one token (``"extend"``: the new key is stored
and all keys are read from the cache).  In a group that keeps a window of positions in a
ring, a step's keys are stored only after the step's attention has read the positions
they overwrite.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..tracing import ranged
from .base import BuildContext, KVRequest, Mixer, ParamSpec, register_part
from .norms import RMSNorm


class GQAAttention(Mixer):
    def __init__(
        self,
        ctx: BuildContext,
        prefix: str,
        n_heads: int,
        n_kv_heads: int,
        head_dim: int,
        qk_norm_eps: Optional[float] = None,
        position: Optional[str] = None,
        window: int = 0,
        own_kv: bool = True,
        scale: Optional[float] = None,
        names: Optional[Dict[str, str]] = None,
    ):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads evenly")
        self.ctx = ctx
        self.hidden = ctx.hidden_size
        self.n_heads, self.n_kv_heads, self.head_dim = int(n_heads), int(n_kv_heads), int(head_dim)
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv_heads * self.head_dim
        self.window = int(window or 0)
        self.own_kv = bool(own_kv)
        self.scale = float(scale) if scale is not None else float(self.head_dim) ** -0.5
        self.qk_norm_eps = qk_norm_eps
        n = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.pos = None
        if position is not None:
            try:
                self.pos = ctx.positions[position]
            except KeyError:
                raise ValueError(f"attention at {prefix!r} names unknown position encoding {position!r}") from None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm_w = self.k_norm_w = None

    # -- parameters ---------------------------------------------------------
    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {
            self.names["q"]: ParamSpec((self.q_dim, self.hidden)),
            self.names["o"]: ParamSpec((self.hidden, self.q_dim)),
        }
        if self.own_kv:
            s[self.names["k"]] = ParamSpec((self.kv_dim, self.hidden))
            s[self.names["v"]] = ParamSpec((self.kv_dim, self.hidden))
        if self.qk_norm_eps is not None:
            s[self.names["q_norm"]] = ParamSpec((self.head_dim,), role="norm", init="one_plus_normal")
            if self.own_kv:
                s[self.names["k_norm"]] = ParamSpec((self.head_dim,), role="norm", init="one_plus_normal")
        return s

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        # q, k and v rows in one matrix: one product per token instead of three
        # (the reference runs three, on three streams, src/transformer.cpp:517-533).
        parts = [tensors.pop(self.names["q"])]
        if self.own_kv:
            parts += [tensors.pop(self.names["k"]), tensors.pop(self.names["v"])]
        self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0].contiguous()
        self.w_o = tensors.pop(self.names["o"]).contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm_w = tensors.pop(self.names["q_norm"])
            if self.own_kv:
                self.k_norm_w = tensors.pop(self.names["k_norm"])

    takes_pending_norm = True       # x goes into K.linear first, and nowhere else

    @property
    def captures_start(self) -> bool:
        # the kernels read the batch's device side only; a position encoding that works on q and k
        # itself is somebody else's code
        return self.pos is None or self.pos.rotary_tables() is not None

    def check_kernels(self, dtype) -> None:
        from ..kernels import attention
        attention.check_supported(self.n_heads, self.n_kv_heads, self.head_dim, dtype)

    def memory_request(self):
        if not self.own_kv:
            return None
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        # only the split of a sequence's keys over blocks looks at the planned length and at how many sequences are real
        return K.attention_decode_plan(n_seq, self.n_heads, self.n_kv_heads, self.head_dim, self.window, plan_len, dtype, device, n_live)

    # -- one step -----------------------------------------------------------
    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if mem is None or not hasattr(mem, "k_pages"):
            raise RuntimeError("attention needs key/value memory; the schedule gave it none")
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if (mem.n_kv_heads, mem.head_dim) != (nkv, hd):
            raise RuntimeError(
                f"attention with {nkv} kv heads of {hd} was given memory for "
                f"{mem.n_kv_heads} kv heads of {mem.head_dim}"
            )
        M = x.shape[0]
        with ranged(batch, "mixer.qkv"):
            qkv = K.linear(x, self.w_qkv)
        q = qkv[:, : self.q_dim].view(M, nh, hd)
        if self.own_kv:
            k = qkv[:, self.q_dim : self.q_dim + self.kv_dim].view(M, nkv, hd)
            v = qkv[:, self.q_dim + self.kv_dim :].view(M, nkv, hd)
        else:
            k = v = None
        with ranged(batch, "mixer.attention"):
            a = self._attend(q, k, v, batch, mem, shared)
        with ranged(batch, "mixer.out"):
            # unless the attention's own last kernel waited for the SMs to drain, this product does
            return K.linear(a.view(M, self.q_dim), self.w_o, late_start=not batch.drained_after_attention)

    def _attend(self, q, k, v, batch, mem, shared) -> torch.Tensor:
        """Per-head norm, position encoding, cache store and attention: q[M, heads, d] -> [M, heads, d]."""
        tables = self.pos.rotary_tables() if self.pos is not None else None
        if batch.mode == "extend" and (self.pos is None or tables is not None):
            # one token each: norm, rotation, cache store and attention from the projection's output
            return K.attention_decode_step(q, k, v, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0, tables, mem,
                                           self.scale, self.window, batch)
        # In a ring, a long enough run of new keys overwrites positions that the run's first
        # queries still read: such a step stores after its attention.
        store_first = self.own_kv and not (batch.mode == "mixed" and mem.ring_rows > 0)
        if self.pos is not None and tables is None:
            # a position encoding without rotary tables works on q and k itself:
            # norms, then the part's own encoding, then the store
            K.qk_norm_rope_store(q, k, None, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0,
                                 None, batch, None)
            self.pos.apply(q, k, batch.tok_pos)
            if store_first:
                K.qk_norm_rope_store(None, k, v, None, None, 0.0, None, batch, mem)
        else:
            K.qk_norm_rope_store(q, k, v, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0,
                                 tables, batch, mem if store_first else None)
        if batch.mode == "extend":
            return K.attention_decode(q, mem, self.scale, self.window, batch)
        if self.own_kv:
            shared["k_new"], shared["v_new"] = k, v
        else:
            k, v = shared["k_new"], shared["v_new"]
        if batch.mode == "start":
            a = K.attention_prefill(q, k, v, self.scale, self.window, batch)
        else:
            a = K.attention_chunk(q, k, v, mem, self.scale, self.window, batch)
        if self.own_kv and not store_first:
            def store(k=k, v=v):
                K.qk_norm_rope_store(None, k, v, None, None, 0.0, None, batch, mem)
            if "deferred" in shared:        # entries that borrow this memory still have to read it
                shared["deferred"].append(store)
            else:
                store()
        return a


register_part("mixer", "gqa_attention", GQAAttention)

"""Arrangement of a layer's parts.

Pre-norm residual block, as the reference runs it (src/transformer.cpp:513, :578,
:583, :618): a = mixer(norm_in(h)); h <- h + a; m = ffn(norm_post(h)); h <- h + m.
The block takes and returns the hidden state as a pair (h, delta) with the pending
sum h + delta not yet formed, so that each sum is done inside the norm that follows
it (the next block's, or the model's final norm).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from .base import Block, BuildContext, ParamSpec, PartSpec, build_part, register_part


class PreNormBlock(Block):
    def __init__(self, ctx: BuildContext, prefix: str, norm: PartSpec, mixer: PartSpec,
                 feed_forward: PartSpec, names: Optional[Dict[str, str]] = None):
        n = {"norm_in": "input_layernorm.", "norm_post": "post_attention_layernorm.",
             "mixer": "self_attn.", "feed_forward": "mlp."}
        n.update(names or {})
        self.norm_in = build_part("norm", norm, ctx, prefix + n["norm_in"])
        self.norm_post = build_part("norm", norm, ctx, prefix + n["norm_post"])
        self.mixer = build_part("mixer", mixer, ctx, prefix + n["mixer"])
        self.feed_forward = build_part("feed_forward", feed_forward, ctx, prefix + n["feed_forward"])
        self._children = (self.norm_in, self.norm_post, self.mixer, self.feed_forward)

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for c in self._children:
            out.update(c.param_specs())
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for c in self._children:
            c.bind(tensors)

    def check_kernels(self, dtype) -> None:
        for c in self._children:
            c.check_kernels(dtype)

    @property
    def captures_start(self) -> bool:
        return bool(self.mixer.captures_start and self.feed_forward.captures_start)

    def forward(self, h, delta, batch, mem, shared):
        trace = getattr(batch, "trace", None)
        if trace is not None and trace.active:
            # the two stages the reference times per layer (src/transformer.cpp:363, :428, :511, :595)
            with trace.range("layer.attn_block"):
                h, a = self._mix(h, delta, batch, mem, shared)
            with trace.range("layer.mlp_block"):
                return self._feed(h, a, batch)
        h, a = self._mix(h, delta, batch, mem, shared)
        return self._feed(h, a, batch)

    def _mix(self, h, delta, batch, mem, shared):
        # h += delta (if any); x = norm(h) -- at once, or inside the reader's first product
        x = self.norm_in.add_pending(h, delta) if self.mixer.takes_pending_norm else self.norm_in.add_forward(h, delta)
        a = self.mixer.forward(x, batch, mem, shared)
        if isinstance(x, K.PendingNorm):
            h = x.hidden()
        return h, a

    def _feed(self, h, a, batch):
        # h += a; x = norm(h)
        x = self.norm_post.add_pending(h, a) if self.feed_forward.takes_pending_norm else self.norm_post.add_forward(h, a)
        m = self.feed_forward.forward(x, batch)
        if isinstance(x, K.PendingNorm):
            h = x.hidden()
        return h, m


register_part("block", "prenorm", PreNormBlock)

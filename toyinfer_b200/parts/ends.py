"""The two ends of a model: token embedding and output head.

``TokenEmbedding``: h[t] = E[id_t] * scale.  The reference gathers without a scale
(src/prefill.cu:6-22, src/transformer.cpp:641-644); the scale is a parameter so that an
architecture with an embedding multiplier needs no new part.

``LinearHead``: for the rows whose logits are wanted, the pending residual sum, an
optional final norm, the product with the head matrix into float32
(src/transformer.cpp:460-470, src/decode.cu:251-286), then an optional scale and soft cap
``cap * tanh(x / cap)``.  The matrix is the embedding table when the head is tied (the
reference always ties, src/qwen.cpp:482-483) and a tensor of its own otherwise.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from .base import BuildContext, Embedding, Head, ParamSpec, PartSpec, build_part, register_part


class TokenEmbedding(Embedding):
    def __init__(self, ctx: BuildContext, prefix: str, vocab_size: int, scale: float = 1.0,
                 name: str = "model.embed_tokens.weight"):
        self.vocab_size, self.hidden = int(vocab_size), ctx.hidden_size
        self.scale = float(scale)
        self.name = prefix + name
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.vocab_size, self.hidden))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors.pop(self.name)

    def table(self) -> torch.Tensor:
        return self.weight

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return K.embed(self.weight, token_ids, self.scale)


class LinearHead(Head):
    def __init__(self, ctx: BuildContext, prefix: str, vocab_size: int, norm: Optional[PartSpec] = None,
                 tied: bool = False, scale: float = 1.0, softcap: float = 0.0,
                 name: str = "lm_head.weight", norm_prefix: str = "model.norm."):
        if softcap < 0:
            raise ValueError(f"the head's soft cap must not be negative, got {softcap}")
        self.ctx = ctx
        self.vocab_size, self.hidden = int(vocab_size), ctx.hidden_size
        self.tied = bool(tied)
        self.scale, self.softcap = float(scale), float(softcap)
        self.name = prefix + name
        self.norm = build_part("norm", norm, ctx, prefix + norm_prefix) if norm is not None else None
        self.weight: Optional[torch.Tensor] = None
        if self.tied and ctx.embedding is None:
            raise ValueError("a tied head needs the model's embedding to be built first")

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        if self.norm is not None:
            out.update(self.norm.param_specs())
        if not self.tied:
            out[self.name] = ParamSpec((self.vocab_size, self.hidden))
        return out

    def ignorable_names(self):
        """Tensors a checkpoint may carry for this part without their being used."""
        return (self.name,) if self.tied else ()

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if self.norm is not None:
            self.norm.bind(tensors)
        self.weight = self.ctx.embedding.table() if self.tied else tensors.pop(self.name)

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        x = K.gather_add(h, delta, rows)
        if self.norm is not None:
            x = self.norm.forward(x)
        logits = K.linear(x, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0 or self.softcap > 0.0:
            K.logit_scale_cap(logits, self.scale, self.softcap)
        return logits


register_part("embedding", "token_table", TokenEmbedding)
register_part("head", "linear", LinearHead)

"""Dense gated feed-forward (SwiGLU).

gate = Wg x, up = Wu x, z = up * gate / (1 + exp(-gate)) with the activation and the
product in 32-bit and one rounding, y = Wd z; no bias.  Reference:
src/transformer.cpp:597-617 (order), src/decode.cu:746-764 (activation).  Gate and
up rows are kept in one matrix, row 2i the gate's and row 2i+1 the up's i-th, so that one
product makes both and the activation can run in that product's epilogue.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from .base import BuildContext, FeedForward, ParamSpec, register_part


class SwiGLU(FeedForward):
    def __init__(self, ctx: BuildContext, prefix: str, intermediate_size: int,
                 names: Optional[Dict[str, str]] = None):
        self.hidden = ctx.hidden_size
        self.inter = int(intermediate_size)
        n = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            self.names["gate"]: ParamSpec((self.inter, self.hidden)),
            self.names["up"]: ParamSpec((self.inter, self.hidden)),
            self.names["down"]: ParamSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g = tensors.pop(self.names["gate"])
        u = tensors.pop(self.names["up"])
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden).contiguous()
        del g, u
        self.w_down = tensors.pop(self.names["down"]).contiguous()

    takes_pending_norm = True       # x goes into K.linear_swiglu, and nowhere else
    captures_start = True

    def forward(self, x, batch) -> torch.Tensor:
        z = K.linear_swiglu(x, self.w_gate_up)    # [M, inter]
        return K.linear(z, self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)

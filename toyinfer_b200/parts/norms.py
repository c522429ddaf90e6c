"""RMS normalisation.

y_i = x_i * rsqrt(mean_j(x_j^2) + eps) * w_i, with the sum, the reciprocal square
root and the product in 32-bit and one rounding at the end; the weight multiplies
directly (no 1 + w).  Reference: src/decode.cu:99-125 (one token),
src/prefill.cu:74-94 (rows of a prompt).  The fused form adds the pending residual
first: the reference does that with a separate kernel (src/decode.cu:7-22) and a
copy (src/transformer.cpp:578-583).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from .base import BuildContext, Norm, ParamSpec, register_part


class RMSNorm(Norm):
    def __init__(self, ctx: BuildContext, prefix: str, size: int, eps: float, name: str = "weight"):
        self.size = int(size)
        self.eps = float(eps)
        self.weight_name = prefix + name
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), role="norm", init="one_plus_normal")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, h: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        if delta is None:
            return K.rmsnorm(h, self.weight, self.eps)
        return K.add_rmsnorm(h, delta, self.weight, self.eps)

    def add_pending(self, h: torch.Tensor, delta: Optional[torch.Tensor]):
        pending = K.pending_norm(h, delta, self.weight, self.eps)
        return pending if pending is not None else self.add_forward(h, delta)


register_part("norm", "rmsnorm", RMSNorm)

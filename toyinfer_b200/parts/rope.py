"""Rotary position encoding with half-rotation pairing.

inv_freq_i = theta^(-2i/d) for i < d/2; the pair (x_i, x_{i+d/2}) of a head is
rotated by the angle pos * inv_freq_i:
x_i <- x_i cos - x_{i+d/2} sin,  x_{i+d/2} <- x_{i+d/2} cos + x_i sin.
Reference: src/decode.cu:35-41 (frequencies), src/decode.cu:301-324 and
src/prefill.cu:185-208 (rotation).  The reference evaluates cosf/sinf of a 32-bit
product in every kernel; here the angles are formed once, in 64-bit, into 32-bit
cos and sin tables [max_positions, d/2] that every kernel reads, so that a
position has one angle whichever way the tokens are cut into steps.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import BuildContext, PositionEncoding, register_part


def rotary_tables(dim: int, theta: float, max_positions: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of pos * theta^(-2i/dim), computed in 64-bit, returned as float32."""
    half = dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -(2.0 * i) / dim)
    pos = torch.arange(max_positions, dtype=torch.float64)
    ang = pos[:, None] * inv_freq[None, :]
    return torch.cos(ang).to(torch.float32), torch.sin(ang).to(torch.float32)


class RotaryHalf(PositionEncoding):
    def __init__(self, ctx: BuildContext, prefix: str, dim: int, theta: float, max_positions: int):
        if dim % 2:
            raise ValueError(f"rotary dimension must be even, got {dim}")
        self.dim = int(dim)
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        cos, sin = rotary_tables(self.dim, self.theta, self.max_positions)
        self.cos = cos.to(ctx.device).contiguous()
        self.sin = sin.to(ctx.device).contiguous()

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        return self.cos, self.sin, self.dim


register_part("position", "rotary_half", RotaryHalf)

"""Which matrix-product kernel runs a given shape."""
from __future__ import annotations

import torch

from . import _call, _code, _ptr, _stream
from .lib import library


def run(x, w, out, M, N, K, ldx, ldw) -> None:
    out_f32 = 1 if (out.dtype == torch.float32 and x.dtype != torch.float32) else 0
    _call(library().ti_linear_simt, _ptr(x), _ptr(w), _ptr(out), M, N, K, ldx, ldw, out.stride(0),
          _code(x, "linear"), out_f32, _stream())

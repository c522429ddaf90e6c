"""Which matrix-product kernel runs a given shape.

bfloat16 operands whose rows are 16-byte aligned go to the tcgen05 kernel (the weights play
the 128-row operand when there are at most 64 tokens), or, for up to 8 tokens (16 for small
matrices), to kernels that only stream the weights (CUDA cores for one token, mma.sync beyond); everything else,
and the whole 32-bit engine, runs on the CUDA-core kernels.
"""
from __future__ import annotations

import ctypes

import torch

from . import _call, _code, _ptr, _stream
from .lib import library

# Measured in whole decode steps of a 4B-shaped model at 2,048 positions (ms per step at 1 / 2 / 4 / 8
# sequences, every product of the step through the one kernel): tcgen05 swap-AB kernel 2.80 / 2.75 /
# 2.82 / 3.01, weight-streaming kernel 2.26 / 2.87 / - / -, small-batch mma.sync kernel 2.41 / 2.51 /
# 2.63 / 2.88; at 16 sequences the tcgen05 kernel 3.37 against 3.58.
GEMV_MAX_TOKENS = 1      # one token: a plain read of the weights on the CUDA cores
SKINNY_MAX_TOKENS = 8    # up to this many: mma.sync with both operands loaded straight from global memory
# ... and up to 16 tokens where the matrix is small: the tcgen05 kernel's fixed costs (tensor memory,
# barriers, a split contraction to add up) then weigh more than the second tile of tokens does here.
# Measured alone at 12 and 16 tokens, us, this kernel against tcgen05: 4,096 x 1,024 3.1 / 5.8, 2,048 x 2,048
# 4.4 / 6.6, 6,144 x 2,560 7.2 / 9.1, 6,144 x 4,096 10.3 / 12.0, but 7,168 x 5,120 20.5 / 14.8, 2,560 x 9,728
# 16.4 / 12.6.  In whole decode steps of 9 to 16 sequences only the small shapes keep the gain (0.6B-shaped
# layers 1.53 -> 1.36 ms; with 4B's q/k/v and output projections here too 3.02 -> 3.12, 8B's 4.03 -> 4.24):
# the limits are those of the small shapes.
SKINNY_SMALL_MAX_TOKENS = 16
SKINNY_SMALL_MAX_K = 3072
SKINNY_SMALL_MAX_WEIGHTS = 8_500_000
_tickets = {}
_plans = {}         # (M, N, K, sms) -> (workspace floats, tickets) as ti_linear_tc_plan answers
_sm_counts = {}


def sm_count(device) -> int:
    """Streaming multiprocessors of the device; launch shapes are planned to fill them once."""
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def _tickets_for(device) -> torch.Tensor:
    t = _tickets.get(device)
    if t is None:
        t = _tickets[device] = torch.zeros(4096, dtype=torch.int32, device=device)
    return t


def set_pair_mode(mode: int) -> None:
    """For tests and measurements: 0 the plan decides between one and two SMs per tile, 1 never two,
    2 two wherever there is a tile per pair.  Plans kept from before are forgotten."""
    library().ti_set_gemm_pair_mode(int(mode))
    _plans.clear()


def set_tile_force(bn: int, splits: int = 0) -> None:
    """For measurements: products of more than 64 tokens that do not run on two SMs per tile take tiles of
    ``bn`` weight rows (128 to 256 in steps of 16) and split the contraction ``splits`` ways (0: as planned);
    ``bn = 0`` ends it.  Plans kept from before are forgotten."""
    library().ti_set_gemm_force(int(bn), int(splits))
    _plans.clear()


def set_skinny_rows(rows: int) -> None:
    """For tests: the products of 2 to 8 tokens take groups of ``rows`` weight rows (8 to 16) whatever the
    shape; 0 lets shape and device decide again."""
    library().ti_set_skinny_rows(int(rows))


def tc_eligible(x, w, K, ldx, ldw) -> bool:
    return (x.dtype == torch.bfloat16 and K % 8 == 0 and ldx % 8 == 0 and ldw % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def run(x, w, out, M, N, K, ldx, ldw, gated: bool = False, late_start: bool = False) -> None:
    """``gated``: only for shapes the tensor-core kernel takes (see tc_eligible).  ``late_start``: the
    few-token kernels start only when the kernel before them has finished (csrc/gemm_skinny.cu)."""
    lib = library()
    out_f32 = 1 if (out.dtype == torch.float32 and x.dtype != torch.float32) else 0
    if tc_eligible(x, w, K, ldx, ldw) and M <= GEMV_MAX_TOKENS:
        _call(lib.ti_linear_gemv, _ptr(x), _ptr(w), _ptr(out), M, N, K, ldx, ldw, out.stride(0), out_f32, 1 if gated else 0,
              sm_count(x.device), 1 if late_start else 0, _stream())
        return
    if tc_eligible(x, w, K, ldx, ldw) and (M <= SKINNY_MAX_TOKENS or (
            M <= SKINNY_SMALL_MAX_TOKENS and SKINNY_MAX_TOKENS >= 8 and K <= SKINNY_SMALL_MAX_K and N * K <= SKINNY_SMALL_MAX_WEIGHTS)):
        _call(lib.ti_linear_skinny, _ptr(x), _ptr(w), _ptr(out), M, N, K, ldx, ldw, out.stride(0), out_f32, 1 if gated else 0,
              sm_count(x.device), 1 if late_start else 0, _stream())
        return
    if tc_eligible(x, w, K, ldx, ldw):
        sms = sm_count(x.device)
        plan = _plans.get((M, N, K, sms))
        if plan is None:        # (workspace floats, tiles that need a ticket) of this shape: asked once
            swap, bn, splits, n_tiles = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
            ws = ctypes.c_longlong()
            lib.ti_linear_tc_plan(M, N, K, sms, ctypes.byref(swap), ctypes.byref(bn), ctypes.byref(splits),
                                  ctypes.byref(ws), ctypes.byref(n_tiles))
            if len(_plans) > 4096:
                _plans.clear()
            plan = _plans[(M, N, K, sms)] = (ws.value, n_tiles.value)
        workspace = tickets = None
        if plan[0] > 0:
            workspace = torch.empty(plan[0], dtype=torch.float32, device=x.device)
            # tickets let the last block of a tile add the partial tiles itself; measured faster
            # than the separate reduction kernel the library falls back to without them
            tickets = _tickets_for(x.device)
            if plan[1] > tickets.numel():
                tickets = None
        _call(lib.ti_linear_tc, _ptr(x), _ptr(w), _ptr(out), M, N, K, ldx, ldw, out.stride(0), out_f32, 1 if gated else 0, sms,
              _ptr(workspace), _ptr(tickets), _stream())
        return
    if gated:
        raise RuntimeError("linear: the gated epilogue exists in the tensor-core kernel only")
    _call(lib.ti_linear_simt, _ptr(x), _ptr(w), _ptr(out), M, N, K, ldx, ldw, out.stride(0),
          _code(x, "linear"), out_f32, _stream())

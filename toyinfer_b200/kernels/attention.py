"""Which attention kernel runs a given shape, and the scratch memory of the split
decode kernel."""
from __future__ import annotations

import torch

from . import KernelError, _call, _code, _ptr, _row_stride, _stream
from .gemm import sm_count
from .lib import library


def prefill(q, k, v, out, scale, window, batch) -> None:
    M, nh, hd = q.shape
    qs, ks, vs = _row_stride(q, "q"), _row_stride(k, "k"), _row_stride(v, "v")
    if (q.dtype == torch.bfloat16 and hd in (64, 128) and qs % 8 == 0 and ks % 8 == 0 and vs % 8 == 0
            and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0):
        fn = library().ti_attn_prefill_tc if (hd == 128 and out.stride(0) % 8 == 0) else library().ti_attn_prefill_mma
        _call(fn, _ptr(q), _ptr(k), _ptr(v), _ptr(out), qs, ks, vs, out.stride(0),
              _ptr(batch.cu_new), batch.n_seq, batch.max_new, M, nh, k.shape[1], hd, scale, window, _stream())
        return
    _call(library().ti_attn_prefill_simt, _ptr(q), _ptr(k), _ptr(v), _ptr(out),
          _row_stride(q, "q"), _row_stride(k, "k"), _row_stride(v, "v"), out.stride(0),
          _ptr(batch.cu_new), batch.n_seq, batch.max_new, nh, k.shape[1], hd, scale, window,
          _code(q, "attention_prefill"), _stream())


def decode_splits(n_seq: int, n_kv_heads: int, max_len: int, page: int, sms: int) -> int:
    """Splits along the keys so that the grid has about two blocks per SM, but no split
    shorter than two pages.  Depends only on the batch's padded size and the longest
    length the step was planned for, so that a captured launch stays valid."""
    tiles = max(1, (max_len + page - 1) // page)
    want = max(1, (2 * sms) // max(1, n_seq * n_kv_heads))
    return max(1, min(want, (tiles + 1) // 2, 64))


def decode(q, mem, out, scale, window, batch) -> None:
    B, nh, hd = q.shape
    nkv = mem.n_kv_heads
    span = batch.plan_len if window <= 0 else min(batch.plan_len, window + mem.page_size)
    splits = decode_splits(B, nkv, span, mem.page_size, sm_count(q.device))
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((B, nh, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((B, nh, splits, 2), dtype=torch.float32, device=q.device)
    pt = mem.page_table
    lib = library()
    fn = lib.ti_attn_decode_mma if (q.dtype == torch.bfloat16 and hd in (64, 128)) else lib.ti_attn_decode_simt
    _call(fn, _ptr(q), _row_stride(q, "q"), _ptr(mem.k_pages), _ptr(mem.v_pages),
          _ptr(pt), pt.shape[1], mem.page_size, mem.ring_rows, mem.k_pages.shape[0],
          _ptr(batch.seq_slot), _ptr(batch.seq_len), B, nh, nkv, hd, scale, window, splits,
          _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), _code(q, "attention_decode"), _stream(),
          launches=2 if splits > 1 else 1)

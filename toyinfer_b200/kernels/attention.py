"""Which attention kernel runs a given shape, and the scratch memory of the split
decode kernel."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import KernelError, _call, _code, _ptr, _row_stride, _stream
from .gemm import sm_count
from .lib import library


def check_supported(n_heads: int, n_kv_heads: int, head_dim: int, dtype) -> None:
    """Raises KernelError when no attention kernel of the library takes these sizes: the limits of
    the CUDA-core kernels, which run whatever the tensor-core kernels (bfloat16, heads of 64 or
    128) do not."""
    if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} heads over {n_kv_heads} kv heads")
    if head_dim % 4 or head_dim < 4 or head_dim > 256:
        raise KernelError(f"attention_prefill: head size {head_dim} not supported (multiples of 4 up to 256)")
    group = n_heads // n_kv_heads
    tensor_cores = dtype == torch.bfloat16 and head_dim in (64, 128)
    if not tensor_cores:
        if group * head_dim > 32 * 128:
            raise KernelError(f"attention_decode: {group} query heads per kv head of size {head_dim} exceed this kernel's "
                              f"{32 * 128} outputs per block")
        smem = (group * head_dim + 64 * (head_dim + 1) + 64 * head_dim + group * 64 + 3 * group) * 4
        if smem > 227 * 1024:
            raise KernelError(f"attention_decode: {group} query heads per kv head of size {head_dim} need {smem} bytes "
                              f"of shared memory")


prefer_mma_sync = False      # tests set this to run the `mma.sync` prompt and chunk kernels, which heads of 64 and 128
                             # otherwise reach only when the output's stride does not fit the tcgen05 kernel's stores


def prefill(q, k, v, out, scale, window, batch) -> None:
    M, nh, hd = q.shape
    qs, ks, vs = _row_stride(q, "q"), _row_stride(k, "k"), _row_stride(v, "v")
    if (q.dtype == torch.bfloat16 and hd in (64, 128) and qs % 8 == 0 and ks % 8 == 0 and vs % 8 == 0
            and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0):
        tcgen05 = out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0 and not prefer_mma_sync
        fn = library().ti_attn_prefill_tc if tcgen05 else library().ti_attn_prefill_mma
        _call(fn, _ptr(q), _ptr(k), _ptr(v), _ptr(out), qs, ks, vs, out.stride(0),
              _ptr(batch.cu_new), batch.n_seq, batch.max_new, M, nh, k.shape[1], hd, scale, window, _stream())
        return
    _call(library().ti_attn_prefill_simt, _ptr(q), _ptr(k), _ptr(v), _ptr(out),
          _row_stride(q, "q"), _row_stride(k, "k"), _row_stride(v, "v"), out.stride(0),
          _ptr(batch.cu_new), batch.n_seq, batch.max_new, nh, k.shape[1], hd, scale, window,
          _code(q, "attention_prefill"), _stream())


MAX_CLUSTER = 16     # splits that the tensor-core decode kernel merges itself, as one thread-block cluster


def chunk(q, k, v, mem, out, scale, window, batch) -> None:
    """New tokens after positions that the cache holds: keys below a sequence's start come from
    ``mem``'s pages, the rest from k and v."""
    M, nh, hd = q.shape
    qs, ks, vs = _row_stride(q, "q"), _row_stride(k, "k"), _row_stride(v, "v")
    pt = mem.page_table
    if mem.k_pages.dtype != q.dtype or not mem.k_pages.is_contiguous() or not mem.v_pages.is_contiguous():
        raise KernelError("attention_chunk: the cache pages do not fit these queries")
    cache = (_ptr(mem.k_pages), _ptr(mem.v_pages), _ptr(pt), pt.shape[1], mem.page_size, mem.ring_rows, mem.k_pages.shape[0])
    if (q.dtype == torch.bfloat16 and hd in (64, 128) and mem.page_size == 64 and qs % 8 == 0 and ks % 8 == 0 and vs % 8 == 0
            and out.stride(0) % 2 == 0 and q.data_ptr() % 16 == 0 and k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0
            and mem.k_pages.data_ptr() % 16 == 0 and mem.v_pages.data_ptr() % 16 == 0):
        tcgen05 = out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0 and not prefer_mma_sync
        fn = library().ti_attn_chunk_tc if tcgen05 else library().ti_attn_chunk_mma
        _call(fn, _ptr(q), _ptr(k), _ptr(v), _ptr(out), qs, ks, vs, out.stride(0),
              _ptr(batch.cu_new), _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seq, batch.max_new, M, nh,
              k.shape[1], hd, scale, window, *cache, _stream())
        return
    _call(library().ti_attn_chunk_simt, _ptr(q), _ptr(k), _ptr(v), _ptr(out), qs, ks, vs, out.stride(0),
          _ptr(batch.cu_new), _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seq, batch.max_new, nh,
          k.shape[1], hd, scale, window, *cache, _code(q, "attention_chunk"), _stream())


def decode_splits(n_seq: int, n_kv_heads: int, max_len: int, page: int, sms: int, min_pages: int = 4, most: int = 64,
                  n_live: Optional[int] = None, places: Optional[int] = None) -> int:
    """Splits along the keys so that the grid has about two blocks per SM, but no split
    shorter than ``min_pages`` pages and no more than ``most``.  Depends only on the batch's
    padded size, the number of its sequences that are real (``n_live``; the others hold one
    position) and the longest length the step was planned for; a captured launch is valid for
    steps that give the same answer.

    A step whose long blocks (a real sequence's kv head each) are a few more than the ``places``
    (blocks that run at once; two per SM unless told) leaves most SMs idle while the rest works off a second round: 38 to 52
    sequences of a batch padded to 64 at 8 kv heads.  Their keys are then split after all, into
    blocks short enough to fill the rounds (measured alone, 40 of 64 sequences at 8,192 positions:
    291 us unsplit, 241 in two, 222 in four, 208 at the copy bandwidth; at 2,048: 76, 68, 71, 52;
    56 and more of 64 are best left whole)."""
    tiles = max(1, (max_len + page - 1) // page)
    want = max(1, (2 * sms) // max(1, n_seq * n_kv_heads))
    longest = (tiles + min_pages - 1) // min_pages
    splits = max(1, min(want, longest, most))
    if splits == 1 and n_live is not None and longest >= 2 and most >= 2:
        places, long_blocks = places or 2 * sms, n_live * n_kv_heads
        if places < long_blocks <= 1.45 * places:
            splits = 4 if (tiles >= 128 and long_blocks <= 1.2 * places and min(longest, most) >= 4) else 2
    return splits


_cluster_room: dict = {}


def cluster_room(hd: int, fused: bool, splits: int) -> int:
    """Clusters of ``splits`` blocks of the tensor-core decode kernel that the device holds at once."""
    key = (hd, bool(fused), splits)
    if key not in _cluster_room:
        room = ctypes.c_int(0)
        _call(library().ti_attn_decode_cluster_room, hd, 1 if fused else 0, splits, ctypes.byref(room), launches=0)
        _cluster_room[key] = room.value
    return _cluster_room[key]


# A decode attention kernel with large shared memory leaves the SMs without an L1 for kernels that
# start while its blocks still run (gemm_skinny.cu).  Its combine kernel, when there is one and the
# step is small enough for the few-token products, is therefore started late: only when the
# attention blocks have left the SMs.  Whether that happened is noted on the step's batch
# (``batch.drained_after_attention``); if not, the product that follows starts late itself
# (kernels.linear(late_start=...), which the mixer sets from the batch).


def _combine_late(n_seq: int) -> bool:
    from . import gemm
    return n_seq <= max(gemm.SKINNY_MAX_TOKENS, gemm.GEMV_MAX_TOKENS)


force_merge_mode = None      # tests set 0, 1 or 2 here to choose how the tensor-core kernel's splits meet


def decode_plan(n_seq: int, n_heads: int, n_kv_heads: int, hd: int, max_len: int, page: int, sms: int,
                tensor_cores: bool, fused: bool, n_live: Optional[int] = None) -> tuple:
    """(splits, mode) of a decode step's attention.  mode (csrc/attn_decode_mma.cu): 2 the splits of a
    kv head are one cluster and merge through distributed shared memory (no scratch, no second kernel);
    else through global scratch and a combine kernel, started late (1) or like every kernel (0).

    The cluster form takes splits of two pages and up to 16 blocks, but only when all of the step's
    clusters find room on the device together with some to spare (clusters are placed whole, inside one
    part of the chip: a second round of them costs far more than the merge saves).  Measured on 36 layers
    of 32 heads over 8 at 2,112 positions, ms per step, cluster against scratch: one sequence (8 clusters
    of 16, room for 14) 2.13 / 2.18; two (16 of 16) 2.63 / 2.28; four (32 of 9, room for 30) 2.70 / 2.35,
    (32 of 8, room for 33) 2.73 / 2.35; eight (64 of 4, room for 71) ahead by 1 to 3 %."""
    scratch_mode = 1 if _combine_late(n_seq) else 0
    if tensor_cores and force_merge_mode in (None, 2):
        splits = decode_splits(n_seq, n_kv_heads, max_len, page, sms, min_pages=2, most=MAX_CLUSTER)
        clusters = n_seq * n_kv_heads * ((n_heads // n_kv_heads + 15) // 16)
        if splits >= 2 and (force_merge_mode == 2 or clusters * 1.08 <= cluster_room(hd, fused, splits)):
            return splits, 2
    # (how many blocks of the tensor-core kernel the device holds at once: a cluster of one is a block)
    places = cluster_room(hd, fused, 1) if tensor_cores and n_live is not None and n_live * n_kv_heads > 2 * sms else None
    splits = decode_splits(n_seq, n_kv_heads, max_len, page, sms, n_live=n_live, places=places)
    if tensor_cores and force_merge_mode in (0, 1):
        return splits, force_merge_mode
    return splits, scratch_mode


def decode(q, mem, out, scale, window, batch) -> None:
    B, nh, hd = q.shape
    nkv = mem.n_kv_heads
    span = batch.plan_len if window <= 0 else min(batch.plan_len, window + mem.page_size)
    tensor_cores = q.dtype == torch.bfloat16 and hd in (64, 128)
    splits, mode = decode_plan(B, nh, nkv, hd, span, mem.page_size, sm_count(q.device), tensor_cores, False, batch.n_real_seq)
    part_o = part_ml = None
    if splits > 1 and mode != 2:
        part_o = torch.empty((B, nh, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((B, nh, splits, 2), dtype=torch.float32, device=q.device)
    pt = mem.page_table
    lib = library()
    batch.drained_after_attention = tensor_cores and splits > 1 and mode == 1
    fn = lib.ti_attn_decode_mma if tensor_cores else lib.ti_attn_decode_simt
    extra = (mode,) if tensor_cores else ()
    _call(fn, _ptr(q), _row_stride(q, "q"), _ptr(mem.k_pages), _ptr(mem.v_pages),
          _ptr(pt), pt.shape[1], mem.page_size, mem.ring_rows, mem.k_pages.shape[0],
          _ptr(batch.seq_slot), _ptr(batch.seq_len), B, nh, nkv, hd, scale, window, splits,
          _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), _code(q, "attention_decode"), *extra, _stream(),
          launches=2 if (splits > 1 and mode != 2) else 1)


def decode_fused_eligible(q, k, v, q_w, k_w, tables, mem) -> bool:
    """Whether the decode kernel can take the projection's output as it is (norm, rotation and
    cache store folded in): bfloat16, heads of 64 or 128, a rotation over the whole head."""
    hd = q.shape[2]
    if q.dtype != torch.bfloat16 or hd not in (64, 128) or mem.page_size != 64:
        return False
    if tables is not None and (tables[2] != hd or tables[0].dtype != torch.float32 or tables[0].data_ptr() % 16
                               or tables[1].data_ptr() % 16 or not tables[0].is_contiguous() or not tables[1].is_contiguous()):
        return False
    for t in (q, k, v):
        if t is not None and (t.stride(2) != 1 or t.stride(1) != hd or t.stride(0) % 8 or t.data_ptr() % 16):
            return False
    for w in (q_w, k_w):
        if w is not None and (w.dtype not in (torch.bfloat16, torch.float32) or not w.is_contiguous() or w.data_ptr() % 16):
            return False
    if q_w is not None and k_w is not None and q_w.dtype != k_w.dtype:
        return False
    return mem.k_pages.dtype == torch.bfloat16 and mem.k_pages.is_contiguous()


def decode_fused(q, k, v, q_w, k_w, eps, tables, mem, out, scale, window, batch) -> None:
    B, nh, hd = q.shape
    nkv = mem.n_kv_heads
    span = batch.plan_len if window <= 0 else min(batch.plan_len, window + mem.page_size)
    splits, mode = decode_plan(B, nh, nkv, hd, span, mem.page_size, sm_count(q.device), True, True, batch.n_real_seq)
    part_o = part_ml = None
    if splits > 1 and mode != 2:
        part_o = torch.empty((B, nh, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((B, nh, splits, 2), dtype=torch.float32, device=q.device)
    batch.drained_after_attention = splits > 1 and mode == 1
    cos = sin = None
    max_pos = 0
    if tables is not None:
        cos, sin, _ = tables
        max_pos = cos.shape[0]
        if batch.max_pos_after > max_pos:
            raise KernelError(f"attention_decode: position {batch.max_pos_after - 1} is beyond the rotary tables' {max_pos}")
    w = q_w if q_w is not None else k_w
    pt = mem.page_table
    _call(library().ti_attn_decode_fused, _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0) if k is not None else 0,
          v.stride(0) if v is not None else 0, _ptr(q_w), _ptr(k_w), 1 if (w is not None and w.dtype == torch.float32) else 0,
          float(eps), _ptr(cos), _ptr(sin), max_pos, _ptr(mem.k_pages), _ptr(mem.v_pages), _ptr(pt), pt.shape[1],
          mem.page_size, mem.ring_rows, mem.k_pages.shape[0], _ptr(batch.seq_slot), _ptr(batch.seq_len), B, nh, nkv, hd,
          scale, window, splits, _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), _code(q, "attention_decode"),
          mode, _stream(), launches=2 if (splits > 1 and mode != 2) else 1)

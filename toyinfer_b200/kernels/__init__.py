"""Python face of the CUDA kernels: one function per operation.

Each function checks shapes, dtypes and devices, allocates its output with torch and
calls the C entry point of the shared library on the current CUDA stream.  There is no
other implementation behind these names: a tensor that is not on a CUDA device, or a
library that cannot be built and loaded, is an error.

The parts of a model call these through the module (``K.linear(...)``), never through
names imported from it, so that the functions can be looked up at call time.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .lib import KernelError, library  # noqa: F401

_CODES = {torch.float32: 0, torch.bfloat16: 1}
launch_count = 0   # kernels launched through this module since import (for measurements)


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]):
    """The tensor's address as ctypes takes it for a pointer argument: an integer, or None for null
    (no object is built: a prompt step passes 1,700 pointers)."""
    return None if t is None else t.data_ptr()


# The current stream's handle, asked for at every launch: torch.cuda.current_stream() builds a Python
# object on the way (a prompt step of 36 layers asks 290 times: 2 ms of its 8 ms on the host), the
# raw query behind it does not.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors, what: str) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(f"{what}: tensors must be on a CUDA device (got {t.device}); there is no CPU path")


def _call(fn, *args, launches: int = 1) -> None:
    global launch_count
    rc = fn(*args)
    if rc != 0:
        raise KernelError(library().ti_last_error().decode("utf-8", "replace"))
    launch_count += launches


def _i32(t: torch.Tensor, what: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what}: expected a contiguous int32 tensor, got {t.dtype}")
    return t


def _row_stride(t: torch.Tensor, what: str) -> int:
    """Elements between consecutive tokens of a [M, heads, dim] or [M, N] view whose
    trailing dimensions are dense."""
    if t.dim() == 3:
        if t.stride(2) != 1 or t.stride(1) != t.shape[2]:
            raise KernelError(f"{what}: heads of a token must be dense")
    elif t.dim() == 2:
        if t.stride(1) != 1:
            raise KernelError(f"{what}: rows must be dense")
    else:
        raise KernelError(f"{what}: expected 2 or 3 dimensions")
    return t.stride(0)


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[m] = table[ids[m]] * scale (a copy when the scale is 1)."""
    _need_cuda(table, ids, what="embed")
    _i32(ids, "embed ids")
    V, H = table.shape
    out = torch.empty((ids.numel(), H), dtype=table.dtype, device=table.device)
    _call(library().ti_embed, _ptr(table), _ptr(ids), _ptr(out), ids.numel(), H, V, float(scale), _code(table, "embed"), _stream())
    return out


def logit_scale_cap(logits: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on float32 logits [rows, vocab]: times ``scale``, then with ``cap`` > 0 the soft
    cap ``cap * tanh(x / cap)``.  Returns its argument."""
    _need_cuda(logits, what="logit_scale_cap")
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logit_scale_cap: expected float32 [rows, vocab] with dense rows")
    R, V = logits.shape
    _call(library().ti_logit_scale_cap, _ptr(logits), logits.stride(0), R, V, float(scale), float(cap), _stream())
    return logits


def _wcode(x: torch.Tensor, w: torch.Tensor, what: str) -> int:
    wc = _code(w, what + " weight")
    if x.dtype == torch.float32 and wc != 0:
        raise KernelError(f"{what}: float32 rows need a float32 weight")
    return wc


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    _need_cuda(x, w, what="rmsnorm")
    M, H = x.shape
    if w.shape != (H,) or not w.is_contiguous():
        raise KernelError(f"rmsnorm: weight {tuple(w.shape)} does not fit rows of {H}")
    stride = _row_stride(x, "rmsnorm")
    out = torch.empty((M, H), dtype=x.dtype, device=x.device)
    _call(library().ti_rmsnorm, _ptr(x), _ptr(None), _ptr(w), _ptr(out), M, H, stride, float(eps),
          _code(x, "rmsnorm"), _wcode(x, w, "rmsnorm"), _stream())
    return out


def add_rmsnorm(h: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """h <- h + delta in place (rounded once); returns rmsnorm(h) * w."""
    _need_cuda(h, delta, w, what="add_rmsnorm")
    M, H = h.shape
    if delta.shape != h.shape or delta.dtype != h.dtype or not h.is_contiguous() or not delta.is_contiguous():
        raise KernelError("add_rmsnorm: h and delta must be dense tensors of one shape and dtype")
    if w.shape != (H,) or not w.is_contiguous():
        raise KernelError(f"add_rmsnorm: weight {tuple(w.shape)} does not fit rows of {H}")
    out = torch.empty_like(h)
    _call(library().ti_rmsnorm, _ptr(h), _ptr(delta), _ptr(w), _ptr(out), M, H, H, float(eps),
          _code(h, "add_rmsnorm"), _wcode(h, w, "add_rmsnorm"), _stream())
    return out


class PendingNorm:
    """An input that is not formed yet: rmsnorm(h + delta) * weight (delta may be None).

    ``linear`` and ``linear_swiglu`` take it in place of a tensor.  For one bfloat16 token the
    product's kernel forms the input itself, in every block, and the step has a kernel less;
    otherwise ``tensor()`` runs the norm kernel.  Either way the sum h + delta exists afterwards:
    ``hidden()`` returns it (h itself, updated in place, or a new tensor).  Made by
    ``pending_norm``, which says first whether the product can use it.
    """

    def __init__(self, h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
        self.h, self.delta, self.weight, self.eps = h, delta, weight, float(eps)
        self._x: Optional[torch.Tensor] = None
        self._hidden: Optional[torch.Tensor] = None

    shape = property(lambda self: self.h.shape)
    dtype = property(lambda self: self.h.dtype)
    device = property(lambda self: self.h.device)

    def tensor(self) -> torch.Tensor:
        """The normalised input as a tensor (the norm kernel runs once)."""
        if self._x is None:
            if self._hidden is not None:            # a product has formed the sum already
                self._x = rmsnorm(self._hidden, self.weight, self.eps)
            elif self.delta is None:
                self._x = rmsnorm(self.h, self.weight, self.eps)
                self._hidden = self.h
            else:
                self._x = add_rmsnorm(self.h, self.delta, self.weight, self.eps)
                self._hidden = self.h
        return self._x

    def hidden(self) -> torch.Tensor:
        """h + delta, rounded once."""
        if self._hidden is None:
            self.tensor()
        return self._hidden


def pending_norm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float) -> Optional[PendingNorm]:
    """A PendingNorm if a product can form this input itself (one bfloat16 token on a CUDA device,
    dense, rows of a multiple of 8 up to 24,576 elements), else None."""
    from . import gemm
    if not (h.is_cuda and h.dtype == torch.bfloat16 and h.dim() == 2 and h.is_contiguous() and weight.is_contiguous()):
        return None
    M, H = h.shape
    if M < 1 or M > gemm.GEMV_MAX_TOKENS or M != 1 or H % 8 or H > 24576 or weight.shape != (H,):
        return None
    if weight.dtype not in (torch.bfloat16, torch.float32):
        return None
    if delta is not None and (delta.shape != h.shape or delta.dtype != h.dtype or not delta.is_contiguous()):
        return None
    return PendingNorm(h, delta, weight, eps)


def _linear_pending(x: PendingNorm, w: torch.Tensor, gated: bool) -> Optional[torch.Tensor]:
    """The product with the norm inside, or None if this weight does not allow it."""
    from . import gemm
    h = x.h
    H = h.shape[1]
    if x._x is not None or x._hidden is not None or w.dtype != torch.bfloat16 or w.dim() != 2 or w.shape[1] != H:
        return None
    ldw = w.stride(0)
    if w.stride(1) != 1 or ldw % 8 or w.data_ptr() % 16 or h.shape[0] > gemm.GEMV_MAX_TOKENS:
        return None
    if any(t is not None and t.data_ptr() % 16 for t in (h, x.delta, x.weight)):
        return None
    N = w.shape[0]
    out = torch.empty((1, N // 2 if gated else N), dtype=h.dtype, device=h.device)
    h_out = torch.empty_like(h) if x.delta is not None else None
    _call(library().ti_linear_gemv_normed, _ptr(h), _ptr(x.delta), _ptr(x.weight), 1 if x.weight.dtype == torch.float32 else 0,
          x.eps, _ptr(h_out), _ptr(w), _ptr(out), N, H, ldw, 1 if gated else 0, gemm.sm_count(h.device), _stream())
    x._hidden = h_out if h_out is not None else h
    return out


def gather_add(h: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
    """out[r] = h[rows[r]] + delta[rows[r]] (delta may be None)."""
    _need_cuda(h, delta, rows, what="gather_add")
    _i32(rows, "gather_add rows")
    M, H = h.shape
    if not h.is_contiguous() or (delta is not None and (delta.shape != h.shape or not delta.is_contiguous()
                                                        or delta.dtype != h.dtype)):
        raise KernelError("gather_add: h and delta must be dense tensors of one shape and dtype")
    out = torch.empty((rows.numel(), H), dtype=h.dtype, device=h.device)
    _call(library().ti_gather_add, _ptr(h), _ptr(delta), _ptr(rows), _ptr(out), rows.numel(), H, M,
          _code(h, "gather_add"), _stream())
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           late_start: bool = False) -> torch.Tensor:
    """x[M, K] times w[N, K] transposed -> [M, N]; 32-bit accumulation.  ``out_dtype`` may
    ask for float32 results from bfloat16 operands (the head).  ``late_start``: a hint that x
    comes from a kernel with large shared memory whose blocks may still be on the SMs; the
    few-token kernels then start only when it has finished (a matter of speed, not of
    results: csrc/gemm_skinny.cu).  x may be a PendingNorm."""
    if isinstance(x, PendingNorm):
        out = _linear_pending(x, w, gated=False) if out_dtype in (None, x.dtype) else None
        if out is not None:
            return out
        x = x.tensor()
    _need_cuda(x, w, what="linear")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError(f"linear: shapes {tuple(x.shape)} and {tuple(w.shape)} do not contract")
    if x.dtype != w.dtype:
        raise KernelError(f"linear: activations are {x.dtype} but the weight is {w.dtype}")
    M, K = x.shape
    N = w.shape[0]
    out_dtype = out_dtype or x.dtype
    if out_dtype not in (x.dtype, torch.float32):
        raise KernelError(f"linear: output dtype {out_dtype} is not supported for {x.dtype} operands")
    ldx, ldw = _row_stride(x, "linear x"), _row_stride(w, "linear w")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    from . import gemm
    gemm.run(x, w, out, M, N, K, ldx, ldw, late_start=bool(late_start))
    return out


def swiglu(gu: torch.Tensor, pairs: bool = False) -> torch.Tensor:
    """up * gate / (1 + exp(-gate)).  gu[M, 2*I] holds gate in its first I columns and up in
    the rest, or with ``pairs`` gate_i and up_i side by side."""
    _need_cuda(gu, what="swiglu")
    M, two_i = gu.shape
    if two_i % 2 or not gu.is_contiguous():
        raise KernelError("swiglu: expected a dense [M, 2*I] tensor")
    out = torch.empty((M, two_i // 2), dtype=gu.dtype, device=gu.device)
    _call(library().ti_swiglu, _ptr(gu), _ptr(out), M, two_i // 2, 1 if pairs else 0, _code(gu, "swiglu"), _stream())
    return out


def linear_swiglu(x: torch.Tensor, w_pairs: torch.Tensor) -> torch.Tensor:
    """x[M, K] times w_pairs[2*I, K] (rows gate_0, up_0, gate_1, up_1, ...) followed by the
    gated activation -> [M, I].  The activation runs in the product's epilogue where the
    tensor-core kernel takes the shape, else as a kernel of its own.  x may be a PendingNorm."""
    if isinstance(x, PendingNorm):
        out = _linear_pending(x, w_pairs, gated=True) if w_pairs.dim() == 2 and w_pairs.shape[0] % 2 == 0 else None
        if out is not None:
            return out
        x = x.tensor()
    _need_cuda(x, w_pairs, what="linear_swiglu")
    if x.dim() != 2 or w_pairs.dim() != 2 or x.shape[1] != w_pairs.shape[1] or w_pairs.shape[0] % 2:
        raise KernelError(f"linear_swiglu: shapes {tuple(x.shape)} and {tuple(w_pairs.shape)} do not fit")
    if x.dtype != w_pairs.dtype:
        raise KernelError(f"linear_swiglu: activations are {x.dtype} but the weight is {w_pairs.dtype}")
    from . import gemm
    M, K = x.shape
    N = w_pairs.shape[0]
    ldx, ldw = _row_stride(x, "linear x"), _row_stride(w_pairs, "linear w")
    if gemm.tc_eligible(x, w_pairs, K, ldx, ldw):
        out = torch.empty((M, N // 2), dtype=x.dtype, device=x.device)
        gemm.run(x, w_pairs, out, M, N, K, ldx, ldw, gated=True)
        return out
    return swiglu(linear(x, w_pairs), pairs=True)


def qk_norm_rope_store(q, k, v, q_w, k_w, eps, tables, batch, mem) -> None:
    """In place on the views q[M, heads, d], k[M, kv_heads, d]: per-head RMS norm (when a
    weight is given), rotation by the cos/sin ``tables`` (when given), and the store of k and
    v[M, kv_heads, d] into ``mem``'s pages (when given).  Any of q, k, v may be None."""
    ref = q if q is not None else k if k is not None else v
    if ref is None:
        return
    _need_cuda(q, k, v, q_w, k_w, what="qk_norm_rope_store")
    M, hd = ref.shape[0], ref.shape[2]
    nh = q.shape[1] if q is not None else 0
    nkv = k.shape[1] if k is not None else (v.shape[1] if v is not None else 0)
    for t in (q, k, v):
        if t is not None and (t.dtype != ref.dtype or t.shape[0] != M or t.shape[2] != hd):
            raise KernelError("qk_norm_rope_store: q, k and v must agree in tokens, head size and dtype")
    w_f32 = 0
    for wt in (q_w, k_w):
        if wt is not None:
            if wt.shape != (hd,) or not wt.is_contiguous():
                raise KernelError(f"qk_norm_rope_store: norm weight {tuple(wt.shape)} does not fit heads of {hd}")
            w_f32 = 1 if wt.dtype == torch.float32 else 0
            if wt.dtype not in (ref.dtype, torch.float32):
                raise KernelError("qk_norm_rope_store: norm weight dtype must be the rows' or float32")
    if q_w is not None and k_w is not None and q_w.dtype != k_w.dtype:
        raise KernelError("qk_norm_rope_store: q and k norm weights differ in dtype")
    cos = sin = None
    rot, max_pos = 0, 0
    if tables is not None:
        cos, sin, rot = tables
        max_pos = cos.shape[0]
        if cos.dtype != torch.float32 or cos.shape != sin.shape or cos.shape[1] * 2 != rot:
            raise KernelError("qk_norm_rope_store: rotary tables must be float32 [positions, dim/2]")
        if batch.max_pos_after > max_pos:
            raise KernelError(f"qk_norm_rope_store: position {batch.max_pos_after - 1} is beyond the rotary tables' {max_pos}")
    kp = vp = pt = None
    width = page = ring = n_pages = 0
    if mem is not None:
        kp, vp, pt = mem.k_pages, mem.v_pages, mem.page_table
        if kp.dtype != ref.dtype or tuple(kp.shape[1:]) != (nkv, mem.page_size, hd) or not kp.is_contiguous():
            raise KernelError("qk_norm_rope_store: the cache pages do not fit these keys")
        width, page, ring, n_pages = pt.shape[1], mem.page_size, mem.ring_rows, kp.shape[0]
    _call(library().ti_qk_norm_rope_store,
          _ptr(q), _ptr(k), _ptr(v),
          _row_stride(q, "q") if q is not None else 0, _row_stride(k, "k") if k is not None else 0,
          _row_stride(v, "v") if v is not None else 0,
          nh, nkv, hd, _ptr(q_w), _ptr(k_w), w_f32, float(eps),
          _ptr(cos), _ptr(sin), rot, max_pos,
          _ptr(batch.tok_pos), _ptr(batch.tok_seq), _ptr(batch.seq_slot), _ptr(batch.seq_len),
          _ptr(kp), _ptr(vp), _ptr(pt), width, page, ring, n_pages, M, _code(ref, "qk_norm_rope_store"), _stream())


def attention_prefill(q, k, v, scale: float, window: int, batch) -> torch.Tensor:
    """Causal attention among the step's own tokens (every sequence starts at position 0).
    q[M, heads, d], k and v[M, kv_heads, d] -> [M, heads, d]."""
    _need_cuda(q, k, v, what="attention_prefill")
    M, nh, hd = q.shape
    nkv = k.shape[1]
    if k.shape != v.shape or k.shape[0] != M or k.shape[2] != hd or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("attention_prefill: q, k and v do not fit together")
    out = torch.empty((M, nh, hd), dtype=q.dtype, device=q.device)
    from . import attention
    attention.prefill(q, k, v, out, float(scale), int(window), batch)
    return out


def attention_chunk(q, k, v, mem, scale: float, window: int, batch) -> torch.Tensor:
    """Causal attention of a step whose sequences go on from any position by any number of
    tokens: sequence b's new tokens take positions ``seq_start[b]`` onwards; keys and values at
    positions below the start are read from ``mem`` (what earlier steps stored), the others are
    the step's own k and v[M, kv_heads, d] (normed and rotated; whether they are stored yet does
    not matter).  q[M, heads, d] -> [M, heads, d]."""
    _need_cuda(q, k, v, what="attention_chunk")
    M, nh, hd = q.shape
    if k.shape != v.shape or k.shape[0] != M or k.shape[2] != hd or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("attention_chunk: q, k and v do not fit together")
    if (mem.n_kv_heads, mem.head_dim) != (k.shape[1], hd):
        raise KernelError("attention_chunk: the cache does not fit these keys")
    out = torch.empty((M, nh, hd), dtype=q.dtype, device=q.device)
    from . import attention
    attention.chunk(q, k, v, mem, out, float(scale), int(window), batch)
    return out


def attention_decode_plan(n_seq: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int, plan_len: int, dtype, device,
                          n_live: Optional[int] = None):
    """(splits, way of merging them) that a decode step's attention launches with when it is
    planned for ``plan_len`` positions and ``n_live`` of its ``n_seq`` sequences are real: all of
    the launch that depends on those two."""
    from . import attention
    from .gemm import sm_count
    from ..cache.allocators import PAGE
    span = plan_len if window <= 0 else min(plan_len, window + PAGE)
    tensor_cores = dtype == torch.bfloat16 and head_dim in (64, 128)
    return attention.decode_plan(n_seq, n_heads, n_kv_heads, head_dim, span, PAGE, sm_count(device), tensor_cores, True, n_live)


def attention_decode(q, mem, scale: float, window: int, batch) -> torch.Tensor:
    """One query per sequence over the cache (the new token's key already stored).
    q[B, heads, d] -> [B, heads, d]."""
    _need_cuda(q, what="attention_decode")
    B, nh, hd = q.shape
    out = torch.empty((B, nh, hd), dtype=q.dtype, device=q.device)
    from . import attention
    attention.decode(q, mem, out, float(scale), int(window), batch)
    return out


def attention_decode_step(q, k, v, q_w, k_w, eps, tables, mem, scale: float, window: int, batch) -> torch.Tensor:
    """The attention of a step in which every sequence goes on by one token, from the projection's
    output: q[B, heads, d], k and v[B, kv_heads, d] (None for a layer that reads another's memory)
    get their per-head norm (weights q_w, k_w or None) and rotation (``tables`` or None), k and v
    go to the cache, and q attends over it.  One kernel where the decode kernel can do all of it
    (see attention.decode_fused_eligible), else the rotate-and-store kernel and then the attention.
    q, k and v may be changed in place."""
    _need_cuda(q, k, v, q_w, k_w, what="attention_decode_step")
    from . import attention
    if attention.decode_fused_eligible(q, k, v, q_w, k_w, tables, mem):
        B, nh, hd = q.shape
        if k is not None and (k.shape != v.shape or k.shape[0] != B or k.shape[2] != hd or k.shape[1] != mem.n_kv_heads):
            raise KernelError("attention_decode_step: k and v do not fit the queries or the cache")
        out = torch.empty((B, nh, hd), dtype=q.dtype, device=q.device)
        attention.decode_fused(q, k, v, q_w, k_w, float(eps), tables, mem, out, float(scale), int(window), batch)
        return out
    qk_norm_rope_store(q, k, v, q_w, k_w, eps, tables, batch, mem if k is not None else None)
    return attention_decode(q, mem, scale, window, batch)


_argmax_scratch = {}


def argmax(logits: torch.Tensor) -> torch.Tensor:
    _need_cuda(logits, what="argmax")
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax: expected float32 [rows, vocab] with dense rows")
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # scratch that the kernel leaves zero: a word and a ticket per row, for rows scanned by several blocks
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch[1].numel() < R:
        n = max(1024, 2 * R)
        scratch = _argmax_scratch[logits.device] = (torch.zeros(n, dtype=torch.int64, device=logits.device),
                                                    torch.zeros(n, dtype=torch.int32, device=logits.device))
    from .gemm import sm_count
    _call(library().ti_argmax, _ptr(logits), logits.stride(0), R, V, sm_count(logits.device), _ptr(scratch[0]),
          _ptr(scratch[1]), _ptr(out), _stream())
    return out


two_kernel_sampling = True      # tests clear this to run every setting in its one-block-per-row form


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int,
           keys: torch.Tensor, steps: torch.Tensor) -> torch.Tensor:
    """One draw per row from softmax(logits / temperature) restricted by top_k and top_p.
    ``keys`` (int64) and ``steps`` (int32) make each row's uniform number."""
    _need_cuda(logits, keys, steps, what="sample")
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: expected float32 [rows, vocab] with dense rows")
    R, V = logits.shape
    if keys.dtype != torch.int64 or steps.dtype != torch.int32 or keys.numel() != R or steps.numel() != R:
        raise KernelError("sample: keys must be int64[rows] and steps int32[rows]")
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # the usual settings run as two short kernels over many blocks and need room between them
    lib = library()
    need = int(lib.ti_sample_scratch_bytes(R, V, int(top_k), float(top_p))) if two_kernel_sampling else 0
    scratch = torch.empty((need // 8 + 1,), dtype=torch.int64, device=logits.device) if need > 0 else None
    _call(lib.ti_sample, _ptr(logits), logits.stride(0), R, V, float(temperature), int(top_k), float(top_p),
          ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), _ptr(keys), _ptr(steps), _ptr(out), _ptr(scratch), _stream(),
          launches=1 if need == 0 else 3 if (top_p < 1.0 and not 0 < top_k < V) else 2)
    return out


def uniform_from(seed: int, key: int, step: int) -> float:
    """The uniform number in [0, 1) that ``sample`` draws for (seed, key, step)."""
    return float(library().ti_uniform_from(ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF),
                                           ctypes.c_uint64(key & 0xFFFFFFFFFFFFFFFF),
                                           ctypes.c_uint64(step & 0xFFFFFFFFFFFFFFFF)))


_STATUS = {1: "a wait for a TMA load ran out", 2: "a wait for tensor-core work ran out",
           3: "a wait for a pipeline slot ran out"}


def reset_scratch() -> None:
    """Clears the device scratch that kernels keep between calls and expect to find zero: the
    tickets by which the blocks of a split product find out who is last, and the words and tickets
    of the argmax kernel.  A kernel that gave up on a wait may have left some of them set; every
    later product that met such a ticket would add a stale piece or never write its tile."""
    from . import gemm
    for t in gemm._tickets.values():
        t.zero_()
    for word, tickets in _argmax_scratch.values():
        word.zero_()
        tickets.zero_()


def check_status() -> None:
    """Waits for the device and raises if a kernel gave up on one of its bounded waits
    since the last check (its results are then not to be trusted).  The status word is clear
    afterwards, and so is the scratch that the kernel may have left half-used."""
    v = ctypes.c_int(0)
    if library().ti_read_status(ctypes.byref(v)) != 0:
        raise KernelError(library().ti_last_error().decode("utf-8", "replace"))
    if v.value:
        reset_scratch()
        raise KernelError(f"a kernel reported status {v.value}: {_STATUS.get(v.value, 'unknown')}")


def testing_wait_runs_out(limit: int = 10000) -> bool:
    """Launches the library's test kernel whose one bounded wait (``limit`` polls) is on a barrier
    nothing arrives on.  Returns whether the wait gave up; the status word is then set, as after any
    product kernel's run-out wait.  Faults nothing."""
    from .lib import declare
    fn = declare("ti_test_wait_runs_out", [ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p])
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    _call(fn, int(limit), _ptr(flag), _stream())
    return bool(flag.item())

"""Loads the shared library of CUDA kernels (building it at first use) and declares the
C signatures.  Loading fails loudly: without the library there is nothing to run."""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_longlong, c_uint64, c_void_p

_lib = None
_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


def _declare(lib) -> None:
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    lib.ti_last_error.restype = c_char_p
    lib.ti_last_error.argtypes = []
    sig = {
        "ti_embed": [P, P, P, I, I, I, F, I, P],
        "ti_logit_scale_cap": [P, L, I, I, F, F, P],
        "ti_rmsnorm": [P, P, P, P, I, I, L, F, I, I, P],
        "ti_gather_add": [P, P, P, P, I, I, I, I, P],
        "ti_swiglu": [P, P, I, I, I, I, P],
        "ti_linear_simt": [P, P, P, I, I, I, L, L, L, I, I, P],
        "ti_qk_norm_rope_store": [P, P, P, L, L, L, I, I, I, P, P, I, F, P, P, I, I, P, P, P, P,
                                  P, P, P, I, I, I, I, I, I, P],
        "ti_attn_prefill_simt": [P, P, P, P, L, L, L, L, P, I, I, I, I, I, F, I, I, P],
        "ti_attn_decode_simt": [P, L, P, P, P, I, I, I, I, P, P, I, I, I, I, F, I, I, P, L, P, P, I, P],
        "ti_attn_decode_cluster_room": [I, I, I, P],
        "ti_attn_decode_mma": [P, L, P, P, P, I, I, I, I, P, P, I, I, I, I, F, I, I, P, L, P, P, I, I, P],
        "ti_attn_decode_fused": [P, P, P, L, L, L, P, P, I, F, P, P, I, P, P, P, I, I, I, I, P, P, I, I, I, I, F, I, I,
                                 P, L, P, P, I, I, P],
        "ti_attn_prefill_mma": [P, P, P, P, L, L, L, L, P, I, I, I, I, I, I, F, I, P],
        "ti_attn_prefill_tc": [P, P, P, P, L, L, L, L, P, I, I, I, I, I, I, F, I, P],
        "ti_attn_chunk_simt": [P, P, P, P, L, L, L, L, P, P, P, I, I, I, I, I, F, I, P, P, P, I, I, I, I, I, P],
        "ti_attn_chunk_mma": [P, P, P, P, L, L, L, L, P, P, P, I, I, I, I, I, I, F, I, P, P, P, I, I, I, I, P],
        "ti_attn_chunk_tc": [P, P, P, P, L, L, L, L, P, P, P, I, I, I, I, I, I, F, I, P, P, P, I, I, I, I, P],
        "ti_linear_tc": [P, P, P, I, I, I, L, L, L, I, I, I, P, P, P],
        "ti_linear_gemv": [P, P, P, I, I, I, L, L, L, I, I, I, I, P],
        "ti_linear_skinny": [P, P, P, I, I, I, L, L, L, I, I, I, I, P],
        "ti_linear_gemv_normed": [P, P, P, I, F, P, P, P, I, I, L, I, I, P],
        "ti_linear_tc_plan": [I, I, I, I, P, P, P, P, P],
        "ti_read_status": [P],
        "ti_argmax": [P, L, I, I, I, P, P, P, P],
        "ti_sample": [P, L, I, I, F, I, F, c_uint64, P, P, P, P, P],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.restype = c_int
        fn.argtypes = args
    lib.ti_uniform_from.restype = c_float
    lib.ti_uniform_from.argtypes = [c_uint64, c_uint64, c_uint64]
    lib.ti_sample_scratch_bytes.restype = ctypes.c_longlong
    lib.ti_sample_scratch_bytes.argtypes = [c_int, c_int, c_int, c_float]
    # entry points that later kernels add are declared by their own modules (see declare())


def declare(name: str, argtypes, restype=c_int):
    """Declares one more entry point of the library and returns it."""
    fn = getattr(library(), name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def library():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                from ..csrc.build import BuildError, ensure_built
                try:
                    path = ensure_built()
                except BuildError as exc:
                    raise KernelError(f"the CUDA kernels could not be built: {exc}") from exc
                try:
                    lib = ctypes.CDLL(path)
                except OSError as exc:
                    raise KernelError(f"the CUDA kernel library {path} could not be loaded: {exc}") from exc
                _declare(lib)
                _lib = lib
    return _lib

"""The entry point that allocates nothing (toyinfer_b200/csrc/attn_decode_noalloc.h).

Some users of the library cannot call cudaMalloc where they need decode attention: code
between a framework's memory-pool checkpoints, loops that must not synchronise the device,
plugins with a fixed memory budget.  For them ``ti_attn_decode_noalloc`` keeps the scratch
of the split kernel in a fixed array inside the library.  This test calls it through its
exported C symbol, twice in a row with different shapes (the second call finds the first
call's leftovers in the shared scratch), and compares each result with the usual entry
point's, which gets scratch allocated by the caller.  It also checks that a request larger
than the array is refused.  The file sorts last so that a failure here cannot hide another
test's result in a run that stops at the first failure.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _case(seed, lens, nh, nkv, hd, dtype, window=0):
    from toyinfer_b200.cache.manager import KVView, PAGE, pages_for
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(pages_for(n) for n in lens) + 1
    k = torch.randn(n_pages + 1, nkv, PAGE, hd, generator=g).to(dtype).cuda()
    v = torch.randn(n_pages + 1, nkv, PAGE, hd, generator=g).to(dtype).cuda()
    table = torch.zeros(len(lens) + 1, max(pages_for(n) for n in lens), dtype=torch.int32)
    free = list(range(n_pages, 0, -1))
    for s, n in enumerate(lens):
        for i in range(pages_for(n)):
            table[s, i] = free.pop()
    q = torch.randn(len(lens), nh, hd, generator=g).to(dtype).cuda()
    return dict(q=q, k=k, v=v, table=table.cuda(), slots=torch.arange(len(lens), dtype=torch.int32).cuda(),
                lens=torch.tensor(lens, dtype=torch.int32).cuda(), nh=nh, nkv=nkv, hd=hd, dtype=dtype, window=window)


def _run(lib, c, n_splits, noalloc):
    B = c["q"].shape[0]
    out = torch.empty_like(c["q"])
    code = 0 if c["dtype"] == torch.float32 else 1
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [_ptr(c["q"]), c["q"].stride(0), _ptr(c["k"]), _ptr(c["v"]), _ptr(c["table"]), c["table"].shape[1], 64, 0,
            c["k"].shape[0], _ptr(c["slots"]), _ptr(c["lens"]), B, c["nh"], c["nkv"], c["hd"],
            1.0 / math.sqrt(c["hd"]), c["window"], n_splits, _ptr(out), out.stride(0)]
    if noalloc:
        rc = lib.ti_attn_decode_noalloc(*head, code, stream)
    else:
        part_o = torch.empty(B * c["nh"] * n_splits * c["hd"], dtype=torch.float32, device="cuda")
        part_ml = torch.empty(B * c["nh"] * n_splits * 2, dtype=torch.float32, device="cuda")
        rc = lib.ti_attn_decode_simt(*head, _ptr(part_o), _ptr(part_ml), code, stream)
    torch.cuda.synchronize()
    return rc, out


def test_no_alloc_entry_point_matches_the_usual_one():
    from toyinfer_b200.kernels.lib import library
    lib = library()
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    lib.ti_attn_decode_noalloc.restype = c_int
    lib.ti_attn_decode_noalloc.argtypes = [P, L, P, P, P, I, I, I, I, P, P, I, I, I, I, F, I, I, P, L, I, P]
    tol = {torch.float32: dict(rtol=1e-4, atol=1e-5), torch.bfloat16: dict(rtol=1.6e-2, atol=4e-3)}
    first = _case(1, [300, 64, 1, 129], 8, 2, 64, torch.bfloat16)
    second = _case(2, [70, 500], 6, 3, 32, torch.float32)            # other shapes over the same scratch
    before = torch.cuda.memory_allocated()
    for c, splits in ((first, 4), (second, 3), (first, 2)):
        rc, got = _run(lib, c, splits, noalloc=True)
        assert rc == 0, lib.ti_last_error().decode()
        rc, want = _run(lib, c, splits, noalloc=False)
        assert rc == 0, lib.ti_last_error().decode()
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), **tol[c["dtype"]])
    assert torch.cuda.memory_allocated() <= before + 64 * 1024 * 1024    # only the tensors made here
    # a request beyond the array is refused, with a message, and launches nothing
    big = _case(3, [64] * 40, 64, 8, 128, torch.bfloat16)
    rc, _ = _run(lib, big, 64, noalloc=True)                            # 40 * 64 * 64 * 130 floats > 2^20
    assert rc != 0 and b"scratch" in lib.ti_last_error()
    torch.cuda.synchronize()

"""The entry point that allocates nothing (toyinfer_b200/csrc/attn_decode_noalloc.h).

Some users of the library cannot call cudaMalloc where they need decode attention: code
between a framework's memory-pool checkpoints, loops that must not synchronise the device,
plugins with a fixed memory budget.  For them ``ti_attn_decode_noalloc`` keeps the scratch
of the split kernel in a fixed array inside the library.  This test calls it through its
exported C symbol, twice in a row with different shapes (the second call finds the first
call's leftovers in the shared scratch), and compares each result with the usual entry
point's, which gets scratch allocated by the caller, and with the plain implementation's
attention.  It also checks that a request larger than the array is refused, that the same
request with one split (which needs no scratch) is taken, and a windowed cache (a ring).  The file sorts last so that a failure here cannot hide another
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
    """A cache with random pages; position p of sequence s lives at row p (or p mod the ring) of
    the pages its table row names.  With a window every sequence gets a whole ring of pages."""
    from toyinfer_b200.cache.manager import KVView, PAGE, pages_for
    g = torch.Generator().manual_seed(seed)
    ring = pages_for(window) * PAGE if window else 0
    held = [ring if ring else n for n in lens]
    n_pages = sum(pages_for(n) for n in held) + 1
    k = torch.randn(n_pages + 1, nkv, PAGE, hd, generator=g).to(dtype).cuda()
    v = torch.randn(n_pages + 1, nkv, PAGE, hd, generator=g).to(dtype).cuda()
    table = torch.zeros(len(lens) + 1, max(pages_for(n) for n in held), dtype=torch.int32)
    free = list(range(n_pages, 0, -1))
    for s, n in enumerate(held):
        for i in range(pages_for(n)):
            table[s, i] = free.pop()
    q = torch.randn(len(lens), nh, hd, generator=g).to(dtype).cuda()
    return dict(q=q, k=k, v=v, table=table.cuda(), slots=torch.arange(len(lens), dtype=torch.int32).cuda(),
                lens=torch.tensor(lens, dtype=torch.int32).cuda(), host_lens=list(lens), host_table=table, ring=ring,
                nh=nh, nkv=nkv, hd=hd, dtype=dtype, window=window)


def _plain(c):
    """The plain implementation's attention for the last position of every sequence, from the keys
    and values as they lie in the pages."""
    from plain import qwen3_plain as plain
    k, v, rows = c["k"].cpu(), c["v"].cpu(), []
    for s, n in enumerate(c["host_lens"]):
        lo = max(0, n - c["window"]) if c["window"] else 0
        pos = list(range(lo, n))
        where = [(int(c["host_table"][s, (p % c["ring"] if c["ring"] else p) // 64]), (p % c["ring"] if c["ring"] else p) % 64)
                 for p in pos]
        ks = torch.stack([k[pg, :, ln, :] for pg, ln in where]).double()
        vs = torch.stack([v[pg, :, ln, :] for pg, ln in where]).double()
        q = torch.zeros(len(pos), c["nh"], c["hd"], dtype=torch.float64)
        q[-1] = c["q"][s].cpu().double()
        rounding = None if c["dtype"] == torch.float32 else torch.bfloat16
        rows.append(plain.attention(q, ks, vs, 1.0 / math.sqrt(c["hd"]), 0, rounding)[-1])
    return torch.stack(rows)


def _run(lib, c, n_splits, noalloc):
    B = c["q"].shape[0]
    out = torch.empty_like(c["q"])
    code = 0 if c["dtype"] == torch.float32 else 1
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [_ptr(c["q"]), c["q"].stride(0), _ptr(c["k"]), _ptr(c["v"]), _ptr(c["table"]), c["table"].shape[1], 64, c["ring"],
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
    ringed = _case(4, [300, 129, 100, 64], 4, 1, 48, torch.float32, window=128)   # a window equal to its ring, wrapped
    before = torch.cuda.memory_allocated()
    for c, splits in ((first, 4), (second, 3), (first, 2), (ringed, 2), (second, 1)):
        rc, got = _run(lib, c, splits, noalloc=True)
        assert rc == 0, lib.ti_last_error().decode()
        rc, want = _run(lib, c, splits, noalloc=False)
        assert rc == 0, lib.ti_last_error().decode()
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), **tol[c["dtype"]])
        torch.testing.assert_close(got.cpu().double(), _plain(c), **tol[c["dtype"]])
    assert torch.cuda.memory_allocated() <= before + 64 * 1024 * 1024    # only the tensors made here
    # a request beyond the array is refused, with a message, and launches nothing
    big = _case(3, [64] * 40, 64, 8, 128, torch.bfloat16)
    rc, _ = _run(lib, big, 64, noalloc=True)                            # 40 * 64 * 64 * 130 floats > 2^20
    assert rc != 0 and b"scratch" in lib.ti_last_error()
    torch.cuda.synchronize()
    # the same batch with one split uses no scratch and is taken whatever its size
    rc, got = _run(lib, big, 1, noalloc=True)
    assert rc == 0, lib.ti_last_error().decode()
    torch.testing.assert_close(got.cpu().double(), _plain(big), **tol[torch.bfloat16])

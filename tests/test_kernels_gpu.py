"""Each CUDA kernel alone against the plain implementation's function for the same
part, at sizes other than the tiny models': odd widths, several head sizes, rows that
straddle block boundaries, padded buffers whose tails must stay untouched (the idiom of
the reference's kernel tests, tests/rmsnorm_test_common.h:40-43)."""
from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def tol(dtype):
    # elementwise results: one rounding of the storage type apart at most (plus float32 noise)
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)


def rnd_mode(dtype):
    return None if dtype == torch.float32 else torch.bfloat16


def dev(x, dtype=None):
    return x.to("cuda", dtype) if dtype is not None else x.to("cuda")


def randn(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.fixture(scope="module")
def K():
    import toyinfer_b200.kernels as K
    K.library()
    return K


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [40, 258, 2560, 1030])
def test_embed(K, dtype, H):
    V, M = 77, 19
    table = randn(V, H, seed=1).to(dtype)
    ids = torch.randint(0, V, (M,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    out = K.embed(dev(table), dev(ids))
    assert torch.equal(out.cpu(), table[ids.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,H", [(1, 64), (5, 258), (33, 514), (7, 1030), (3, 2560), (2, 5120)])
def test_rmsnorm_and_fused_sum(K, dtype, M, H):
    x = randn(M, H, seed=3).to(dtype)
    d = randn(M, H, seed=4).to(dtype)
    w = (1 + randn(H, seed=5, scale=0.1)).to(dtype)
    eps = 1e-5
    want = plain.rms_norm(x.double(), w, eps, rnd_mode(dtype))
    got = K.rmsnorm(dev(x), dev(w), eps)
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype))
    # fused: h <- h + d (rounded once), then the norm of the rounded sum
    h = dev(x).clone()
    got = K.add_rmsnorm(h, dev(d), dev(w), eps)
    hs = plain.rnd(x.double() + d.double(), rnd_mode(dtype))
    torch.testing.assert_close(h.cpu().double(), hs, **tol(dtype))
    want = plain.rms_norm(h.cpu().double(), w, eps, rnd_mode(dtype))
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype))


def test_rmsnorm_float32_weight_with_bfloat16_rows(K):
    x = randn(9, 96, seed=6).to(torch.bfloat16)
    w = 1 + randn(96, seed=7, scale=0.1)
    got = K.rmsnorm(dev(x), dev(w), 1e-6)
    want = plain.rms_norm(x.double(), w, 1e-6, torch.bfloat16)
    torch.testing.assert_close(got.cpu().double(), want, **tol(torch.bfloat16))


def test_rmsnorm_strided_rows_and_tail(K):
    buf = torch.full((6, 300), 7.0, dtype=torch.float32, device="cuda")
    x = randn(6, 130, seed=8)
    buf[:, :130] = dev(x)
    w = dev(1 + randn(130, seed=9, scale=0.1))
    got = K.rmsnorm(buf[:, :130], w, 1e-6)
    want = plain.rms_norm(x.double(), w.cpu(), 1e-6)
    torch.testing.assert_close(got.cpu().double(), want, **tol(torch.float32))
    assert torch.all(buf[:, 130:] == 7.0)


@pytest.mark.parametrize("dtype", DT)
def test_gather_add(K, dtype):
    h, d = randn(11, 70, seed=10).to(dtype), randn(11, 70, seed=11).to(dtype)
    rows = torch.tensor([10, 0, 3, 3], dtype=torch.int32)
    got = K.gather_add(dev(h), dev(d), dev(rows))
    want = plain.rnd(h.double()[rows.long()] + d.double()[rows.long()], rnd_mode(dtype))
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype))
    got = K.gather_add(dev(h), None, dev(rows))
    assert torch.equal(got.cpu(), h[rows.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,I", [(1, 128), (5, 200), (3, 9728), (2, 1001)])
def test_swiglu(K, dtype, M, I):
    gu = randn(M, 2 * I, seed=12, scale=2.0).to(dtype)
    got = K.swiglu(dev(gu))
    want = plain.swiglu(gu[:, :I].double(), gu[:, I:].double(), rnd_mode(dtype))
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,I,K_", [(1, 128, 64), (8, 9728, 2560), (5, 200, 96), (70, 144, 80), (300, 1000, 264), (3, 50, 100),
                                    (1300, 1800, 264)])
def test_linear_swiglu(K, dtype, M, I, K_):
    """Gate and up rows side by side in one matrix; the activation in the product's epilogue
    (tensor-core shapes) or in a kernel after it (the rest)."""
    x = randn(M, K_, seed=27).to(dtype)
    wg = randn(I, K_, seed=28, scale=0.08).to(dtype)
    wu = randn(I, K_, seed=29, scale=0.08).to(dtype)
    w = torch.stack([wg, wu], dim=1).reshape(2 * I, K_).contiguous()
    got = K.linear_swiglu(dev(x), dev(w)).cpu().double()
    K.check_status()
    r = rnd_mode(dtype)
    want = plain.swiglu(plain.linear(x.double(), wg, r), plain.linear(x.double(), wu, r), r)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    else:
        torch.testing.assert_close(got, want, rtol=3e-2, atol=4e-3)
    pairs = dev(torch.stack([wg @ x.T, wu @ x.T], dim=1).permute(2, 0, 1).reshape(M, 2 * I).contiguous().to(dtype))
    got2 = K.swiglu(pairs, pairs=True).cpu().double()
    want2 = plain.swiglu(pairs.cpu().double()[:, 0::2], pairs.cpu().double()[:, 1::2], r)
    torch.testing.assert_close(got2, want2, **tol(dtype))


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,N,K_", [(1, 64, 64), (3, 200, 96), (8, 384, 100), (13, 130, 258), (17, 300, 72),
                                    (70, 130, 200), (128, 256, 512), (200, 1000, 264), (5, 2560, 4096)])
def test_linear(K, dtype, M, N, K_):
    x = randn(M, K_, seed=13).to(dtype)
    w = randn(N, K_, seed=14, scale=0.05).to(dtype)
    got = K.linear(dev(x), dev(w))
    want = x.double() @ w.double().T
    if dtype == torch.float32:
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-4, atol=1e-5)
    else:
        torch.testing.assert_close(got.cpu().double(), plain.rnd(want, torch.bfloat16), rtol=1.6e-2, atol=2e-3)
        got32 = K.linear(dev(x), dev(w), out_dtype=torch.float32)
        torch.testing.assert_close(got32.cpu().double(), want, rtol=1e-3, atol=1e-4)


def _planned_shared_tiles(M, N, K_):
    import ctypes
    from toyinfer_b200.kernels.gemm import sm_count
    from toyinfer_b200.kernels.lib import library
    swap, bn, splits, shared, ws = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_longlong()
    library().ti_linear_tc_plan(M, N, K_, sm_count(torch.device("cuda", torch.cuda.current_device())), ctypes.byref(swap),
                                ctypes.byref(bn), ctypes.byref(splits), ctypes.byref(ws), ctypes.byref(shared))
    return shared.value if (not swap.value and splits.value == 1 and bn.value >= 128) else 0


@pytest.mark.parametrize("M,N,K_,f32", [
    (2048, 6144, 2560, False),     # prefill, q/k/v rows of a 4B-shaped layer
    (2048, 2560, 9728, False),     # prefill, down projection (long contraction): one round of tiles 288 wide on pairs of SMs
    (2048, 2560, 4096, False),     # prefill, output projection
    (4096, 2560, 4096, False),     # 2.2 rounds of pairs: tiles shared out by contraction steps
    (2304, 2500, 520, True),       # tiles 320 wide, ragged on both sides (9 x 256 tokens, 8 x 320 > 2,500 columns)
    (2048, 4096, 1032, False),     # tiles 512 wide: two MMAs of 256 columns into one accumulator
    (1000, 1536, 512, False), (777, 3000, 328, True),
    (4741, 520, 264, False),       # more token tiles than one panel of the tile order, the last panel short
    (300, 2560, 4096, False),      # few tiles: the contraction is split
    (100, 2560, 9728, False),      # one row of 20 tiles, four splits
    (256, 2560, 9728, False),      # 40 tiles, three splits: all blocks in one round
    (256, 6144, 2560, False),      # 96 whole tiles, no split
    (192, 19456, 2560, False),     # a pair's tile of 256 tokens a quarter empty, wide tiles in one round
    (1300, 3600, 264, False),      # tiles for a round and a bit, shared out by contraction steps; short parts, ragged K
    (8, 19456, 2560, False),       # decode at batch 8, gate and up rows
    (64, 2560, 9728, False),       # decode at batch 64, split contraction
    (1, 151936, 2560, True),       # head for one row, float32 logits
    (33, 1000, 264, False), (16, 128, 64, False), (65, 136, 72, True), (129, 250, 200, False),
])
def test_linear_tensor_cores_at_model_sizes(K, monkeypatch, M, N, K_, f32):
    """The tcgen05 kernel against a float32 product of the same bfloat16 operands (the kernels
    that otherwise take up to 8 tokens are switched off here)."""
    import toyinfer_b200.kernels.gemm as gemm
    monkeypatch.setattr(gemm, "GEMV_MAX_TOKENS", 0)
    monkeypatch.setattr(gemm, "SKINNY_MAX_TOKENS", 0)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K_, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K_, generator=g, device="cuda") * 0.03).to(torch.bfloat16)
    got = K.linear(x, w, out_dtype=torch.float32 if f32 else None)
    K.check_status()
    if (M, N) in ((4096, 2560), (1300, 3600)):
        assert _planned_shared_tiles(M, N, K_) > 0      # these are here for the tiles that two blocks share
    want = x.float() @ w.float().T
    if f32:
        torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-3)
    else:
        torch.testing.assert_close(got.float(), want.to(torch.bfloat16).float(), rtol=1.6e-2, atol=4e-3)
    # a second call reuses tickets and workspace
    got2 = K.linear(x, w, out_dtype=torch.float32 if f32 else None)
    assert torch.equal(got, got2)


@pytest.mark.parametrize("M,N,K_,f32", [
    (4096, 2560, 4096, False),     # 160 tiles of 256 x 256 for 74 pairs: the last rounds shared out by contraction steps
    (2048, 2560, 4096, False),     # one round of tiles 288 wide on pairs
    (2048, 6144, 2560, False),     # whole tiles in both forms
    (1100, 3000, 328, True),       # ragged on every side; rows past the end in the pair's second block
    (512, 19456, 264, False),      # two token tiles
])
def test_linear_many_tokens_on_one_and_on_two_sms_per_tile(K, M, N, K_, f32):
    """The many-token tcgen05 kernel in both forms, one block per tile of 128 tokens and a pair of blocks
    per tile of 256 (cta_group::2), against a float32 product of the same bfloat16 operands."""
    from toyinfer_b200.kernels import gemm
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(M, K_, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K_, generator=g, device="cuda") * 0.03).to(torch.bfloat16)
    want = x.float() @ w.float().T
    try:
        for mode in (1, 2):
            gemm.set_pair_mode(mode)
            got = K.linear(x, w, out_dtype=torch.float32 if f32 else None)
            K.check_status()
            if f32:
                torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-3)
            else:
                torch.testing.assert_close(got.float(), want.to(torch.bfloat16).float(), rtol=1.6e-2, atol=4e-3)
            assert torch.equal(got, K.linear(x, w, out_dtype=torch.float32 if f32 else None))
    finally:
        gemm.set_pair_mode(0)


@pytest.mark.parametrize("M", [1, 2])
@pytest.mark.parametrize("N,K_", [(6144, 2560), (2560, 9728), (2560, 4096), (19456, 2560), (7, 8), (333, 200), (2, 4104),
                                  (151936, 64), (100, 1024), (30, 20000)])
def test_linear_few_tokens(K, monkeypatch, M, N, K_):
    """The weight-streaming kernel for one or two tokens against a float32 product: bfloat16
    and float32 results, the gated form, odd row counts, contractions shorter than a warp's
    stride, rows shared by several warps (few rows, long contraction), and operands inside
    wider buffers."""
    import toyinfer_b200.kernels.gemm as gemm
    monkeypatch.setattr(gemm, "GEMV_MAX_TOKENS", 2)
    g = torch.Generator(device="cuda").manual_seed(9)
    xb = torch.randn(M, K_ + 16, generator=g, device="cuda").to(torch.bfloat16)
    wb = (torch.randn(N, K_ + 8, generator=g, device="cuda") * 0.03).to(torch.bfloat16)
    x, w = xb[:, 8:8 + K_], wb[:, :K_]
    before = K.launch_count
    got = K.linear(x, w)
    got32 = K.linear(x, w, out_dtype=torch.float32)
    assert K.launch_count == before + 2
    want = x.float() @ w.float().T
    torch.testing.assert_close(got32, want, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(got.float(), want.to(torch.bfloat16).float(), rtol=1.6e-2, atol=4e-3)
    if N % 2 == 0:
        gated = K.linear_swiglu(x, w)
        gate, up = want[:, 0::2], want[:, 1::2]
        torch.testing.assert_close(gated.float(), (up * gate / (1 + torch.exp(-gate))).to(torch.bfloat16).float(),
                                   rtol=3e-2, atol=4e-3)
        assert gated.shape == (M, N // 2)


@pytest.mark.parametrize("norm_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("N,K_,gated,with_delta", [(6144, 2560, False, True), (19456, 2560, True, True), (2560, 5120, False, False),
                                                   (333, 200, False, True), (70, 1032, True, True), (51200, 5120, True, True)])
def test_linear_with_the_norm_inside(K, N, K_, gated, with_delta, norm_dtype):
    """One token's product that forms its own input, rmsnorm(h + delta) * g, against the norm kernel
    followed by the product: the same bits where the norm kernel sums in the same order (bfloat16
    weights, rows longer than 1,024), else within a rounding of the input; and the sum it leaves."""
    g = torch.Generator(device="cuda").manual_seed(11)
    h = torch.randn(1, K_, generator=g, device="cuda").to(torch.bfloat16)
    delta = (torch.randn(1, K_, generator=g, device="cuda") * 0.5).to(torch.bfloat16) if with_delta else None
    gw = (1 + 0.1 * torch.randn(K_, generator=g, device="cuda")).to(norm_dtype)
    w = (torch.randn(N, K_, generator=g, device="cuda") * 0.03).to(torch.bfloat16)
    eps = 1e-5
    h_sum = (h.float() + delta.float()).to(torch.bfloat16) if with_delta else h.clone()
    x = K.rmsnorm(h_sum, gw, eps)
    want = K.linear_swiglu(x, w) if gated else K.linear(x, w)
    pending = K.pending_norm(h.clone(), delta, gw, eps)
    assert pending is not None
    got = K.linear_swiglu(pending, w) if gated else K.linear(pending, w)
    K.check_status()
    assert torch.equal(pending.hidden(), h_sum)
    if norm_dtype == torch.bfloat16 and K_ > 1024:
        assert torch.equal(got, want)
    else:
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    # used a second time, the input is formed by the norm kernel from the sum that exists now
    again = K.linear(pending, w[: N // 2])
    torch.testing.assert_close(again.float(), K.linear(x, w[: N // 2]).float(), rtol=2e-2, atol=2e-2)


def test_pending_norm_is_refused_where_no_product_can_use_it(K):
    h = torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    assert K.pending_norm(h, None, w, 1e-6) is None                       # two tokens
    assert K.pending_norm(h[:1].float(), None, w.float(), 1e-6) is None   # float32
    assert K.pending_norm(h[:1, :60], None, w[:60], 1e-6) is None         # rows of 60 elements: no multiple of 8
    p = K.pending_norm(h[:1], None, w, 1e-6)
    assert p is not None and torch.equal(p.hidden(), h[:1])               # nothing to add: the hidden state is h


@pytest.mark.parametrize("M", [1, 3, 5, 8, 9, 13, 16])
@pytest.mark.parametrize("N,K_", [(6144, 2560), (2560, 9728), (2560, 4096), (19456, 2560), (7, 8), (333, 200), (2, 4104),
                                  (50000, 72), (100, 1024), (30, 20000)])
def test_linear_small_batch(K, monkeypatch, M, N, K_):
    """The small-batch product (operands straight from global memory into mma.sync) against a
    float32 product: bfloat16 and float32 results, the gated form, row counts that are no
    multiple of 16, contractions that are no multiple of 32, rows shared by several warps, and
    operands inside wider buffers."""
    import toyinfer_b200.kernels.gemm as gemm
    monkeypatch.setattr(gemm, "GEMV_MAX_TOKENS", 0)
    monkeypatch.setattr(gemm, "SKINNY_MAX_TOKENS", 16)
    g = torch.Generator(device="cuda").manual_seed(11)
    xb = torch.randn(M, K_ + 16, generator=g, device="cuda").to(torch.bfloat16)
    wb = (torch.randn(N, K_ + 8, generator=g, device="cuda") * 0.03).to(torch.bfloat16)
    x, w = xb[:, 8:8 + K_], wb[:, :K_]
    before = K.launch_count
    got = K.linear(x, w)
    got32 = K.linear(x, w, out_dtype=torch.float32)
    assert K.launch_count == before + 2
    want = x.float() @ w.float().T
    torch.testing.assert_close(got32, want, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(got.float(), want.to(torch.bfloat16).float(), rtol=1.6e-2, atol=4e-3)
    if N % 2 == 0:
        gated = K.linear_swiglu(x, w)
        gate, up = want[:, 0::2], want[:, 1::2]
        torch.testing.assert_close(gated.float(), (up * gate / (1 + torch.exp(-gate))).to(torch.bfloat16).float(),
                                   rtol=3e-2, atol=4e-3)
        assert gated.shape == (M, N // 2)


@pytest.mark.parametrize("rows", [8, 9, 11, 12, 15, 16])
def test_linear_small_batch_with_every_size_of_row_group(K, rows):
    """The product for 2 to 8 tokens takes its weights in groups of 8 to 16 rows, as many as fill the
    device's SMs evenly; here every size is forced in turn, on matrices whose last group is short, plain
    and gated (a gated product's groups are even)."""
    from toyinfer_b200.kernels import gemm
    g = torch.Generator(device="cuda").manual_seed(14)
    try:
        gemm.set_skinny_rows(rows)
        for M, N, K_ in ((8, 2560, 4096), (3, 333, 200), (5, 70, 1032), (2, 16, 64), (7, 9, 72)):
            x = torch.randn(M, K_, generator=g, device="cuda").to(torch.bfloat16)
            w = (torch.randn(N, K_, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
            want = (x.float() @ w.float().T)
            torch.testing.assert_close(K.linear(x, w).float(), want.to(torch.bfloat16).float(), rtol=1.6e-2, atol=4e-3)
            torch.testing.assert_close(K.linear(x, w, out_dtype=torch.float32), want, rtol=1e-3, atol=1e-3)
            if N % 2 == 0:
                gate, up = want[:, 0::2], want[:, 1::2]
                act = up * (gate / (1 + torch.exp(-gate)))
                torch.testing.assert_close(K.linear_swiglu(x, w).float(), act.to(torch.bfloat16).float(), rtol=1.6e-2, atol=4e-3)
            K.check_status()
    finally:
        gemm.set_skinny_rows(0)


@pytest.mark.parametrize("M", [1, 2, 8])
def test_products_back_to_back_read_what_the_kernel_before_wrote(K, M):
    """Kernels are launched so that each may start while the one before it still runs and must
    wait before it reads that kernel's results.  A chain norm -> product -> norm -> product ...
    whose buffers are reused at the same addresses, replayed from a CUDA graph (no gaps between
    the kernels), must give what the same chain gives with a device-wide wait after every kernel."""
    H, N, n = 4096, 2560, 24
    g = torch.Generator(device="cuda").manual_seed(3)
    hs = [torch.randn(M, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(n)]
    wn = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).to(torch.bfloat16)
    w = (torch.randn(N, H, generator=g, device="cuda") * 0.03).to(torch.bfloat16)

    def chain(sync):
        outs = []
        for h in hs:
            x = K.rmsnorm(h, wn, 1e-6)
            if sync:
                torch.cuda.synchronize()
            y = K.linear(x, w)
            if sync:
                torch.cuda.synchronize()
            outs.append(y)
            del x
        return outs

    want = [o.clone() for o in chain(True)]
    chain(False)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = chain(False)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    K.check_status()
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_linear_strided_input_and_tail(K):
    buf = torch.full((9, 500), 3.0, dtype=torch.float32, device="cuda")
    x = randn(9, 120, seed=15)
    buf[:, 100:220] = dev(x)
    w = randn(50, 120, seed=16, scale=0.1)
    got = K.linear(buf[:, 100:220], dev(w))
    torch.testing.assert_close(got.cpu().double(), x.double() @ w.double().T, rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------------------
def make_mem(dtype, n_slots, nkv, hd, pages, window=0, dirty=0.0):
    from toyinfer_b200.cache.manager import KVView, PAGE, pages_for
    ring = pages_for(window) * PAGE if window else 0
    k = torch.full((pages + 1, nkv, PAGE, hd), dirty, dtype=dtype, device="cuda")
    v = torch.full((pages + 1, nkv, PAGE, hd), dirty, dtype=dtype, device="cuda")
    table = torch.zeros((n_slots + 1, pages), dtype=torch.int32, device="cuda")
    return KVView(k, v, table, nkv, hd, window, ring)


def make_batch(mode, slots, starts, news, plan_len=4096, spare_rows=0):
    """With ``spare_rows``, that many token rows of nobody's follow, as in a captured step of fixed size."""
    from toyinfer_b200.engine.batch import BatchBuffers, fill_batch
    toks = [[0] * n for n in news]
    if spare_rows:
        total = sum(news) + spare_rows
        buf = BatchBuffers(len(slots) + 1, total, "cuda")
        return fill_batch(buf, mode, slots, starts, toks, scratch_slot=max(slots) + 1, plan_len=plan_len,
                          total_tok=total, new_bound=max(news) + 5)
    buf = BatchBuffers(len(slots), sum(news), "cuda")
    return fill_batch(buf, mode, slots, starts, toks, scratch_slot=max(slots) + 1, plan_len=plan_len)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (6, 2, 32), (5, 1, 48), (8, 8, 64), (32, 8, 128), (2, 1, 256)])
def test_qk_norm_rope_store(K, dtype, nh, nkv, hd):
    from toyinfer_b200.parts.rope import rotary_tables
    news = [5, 70, 1]
    M = sum(news)
    width = (nh + 2 * nkv) * hd
    qkv = randn(M, width, seed=17).to(dtype)
    qw = (1 + randn(hd, seed=18, scale=0.1)).to(dtype)
    kw = (1 + randn(hd, seed=19, scale=0.1)).to(dtype)
    cos, sin = rotary_tables(hd, 1e4, 128)
    mem = make_mem(dtype, 4, nkv, hd, pages=6, dirty=9.0)
    # slots 2, 0, 3 with pages chosen out of order
    mem.page_table[2, 0] = 5
    mem.page_table[0, 0] = 2
    mem.page_table[0, 1] = 4
    mem.page_table[3, 0] = 1
    batch = make_batch("start", [2, 0, 3], [0, 0, 0], news)
    g = dev(qkv).clone()
    q = g[:, : nh * hd].view(M, nh, hd)
    k = g[:, nh * hd: (nh + nkv) * hd].view(M, nkv, hd)
    v = g[:, (nh + nkv) * hd:].view(M, nkv, hd)
    K.qk_norm_rope_store(q, k, v, dev(qw), dev(kw), 1e-6, (dev(cos), dev(sin), hd), batch, mem)
    pos = [p for n in news for p in range(n)]
    r = rnd_mode(dtype)
    ang = plain.rope_angles(hd, 1e4, pos)
    q0 = qkv[:, : nh * hd].view(M, nh, hd).double()
    k0 = qkv[:, nh * hd: (nh + nkv) * hd].view(M, nkv, hd).double()
    v0 = qkv[:, (nh + nkv) * hd:].view(M, nkv, hd)
    wq = plain.rope(plain.rms_norm(q0, qw, 1e-6, r), ang, r)
    wk = plain.rope(plain.rms_norm(k0, kw, 1e-6, r), ang, r)
    torch.testing.assert_close(q.cpu().double(), wq, **tol(dtype))
    torch.testing.assert_close(k.cpu().double(), wk, **tol(dtype))
    assert torch.equal(v.cpu(), v0)
    # cache contents: sequence 1 (slot 0) spans pages 2 and 4
    kp, vp = mem.k_pages.cpu(), mem.v_pages.cpu()
    assert torch.equal(kp[5, :, :5], k.cpu()[0:5].transpose(0, 1))
    assert torch.equal(kp[2, :, :64], k.cpu()[5:69].transpose(0, 1))
    assert torch.equal(kp[4, :, :6], k.cpu()[69:75].transpose(0, 1))
    assert torch.equal(vp[4, :, :6], v0[69:75].transpose(0, 1))
    assert torch.equal(kp[1, :, :1], k.cpu()[75:76].transpose(0, 1))
    # untouched lines keep the dirty value
    assert torch.all(kp[5, :, 5:] == 9.0) and torch.all(kp[4, :, 6:] == 9.0) and torch.all(kp[3] == 9.0)
    assert torch.all(kp[0] == 9.0)


def test_store_into_ring_keeps_only_the_window(K):
    dtype = torch.float32
    nkv, hd, n = 1, 16, 150
    mem = make_mem(dtype, 1, nkv, hd, pages=1, window=40, dirty=-1.0)   # ring of 64 rows = one page
    mem.page_table[0, 0] = 1
    batch = make_batch("start", [0], [0], [n])
    k = torch.arange(n, dtype=dtype, device="cuda")[:, None, None].expand(n, nkv, hd).contiguous()
    v = (k + 1000).contiguous()
    K.qk_norm_rope_store(None, k, v, None, None, 0.0, None, batch, mem)
    kp = mem.k_pages.cpu()[1, 0, :, 0]
    # positions 86..149 live at row p mod 64
    for p in range(n - 64, n):
        assert kp[p % 64] == p
    assert torch.all(mem.v_pages.cpu()[1, 0, :, 0] == kp + 1000)


# ---------------------------------------------------------------------------
def plain_attention_seq(q, k, v, scale, window, dtype):
    return plain.attention(q.double(), k.double(), v.double(), scale, window, rnd_mode(dtype))


ATT_TOL = {torch.float32: dict(rtol=1e-4, atol=1e-5), torch.bfloat16: dict(rtol=1.6e-2, atol=4e-3)}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (6, 2, 32, 0), (5, 1, 48, 40), (8, 4, 64, 0),
                                               (8, 2, 128, 0), (4, 4, 128, 33), (2, 1, 256, 0)])
def test_attention_prefill(K, dtype, nh, nkv, hd, window):
    news = [1, 100, 32, 33, 7]
    M = sum(news)
    q = randn(M, nh, hd, seed=20).to(dtype)
    k = randn(M, nkv, hd, seed=21).to(dtype)
    v = randn(M, nkv, hd, seed=22).to(dtype)
    batch = make_batch("start", list(range(len(news))), [0] * len(news), news)
    scale = 1.0 / math.sqrt(hd)
    got = K.attention_prefill(dev(q), dev(k), dev(v), scale, window, batch).cpu().double()
    o = 0
    for n in news:
        want = plain_attention_seq(q[o:o + n], k[o:o + n], v[o:o + n], scale, window, dtype)
        torch.testing.assert_close(got[o:o + n], want, **ATT_TOL[dtype])
        o += n


@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, 0), (4, 4, 64, 0), (6, 2, 128, 100), (2, 1, 64, 64), (32, 8, 128, 0)])
def test_attention_prefill_on_views_of_one_buffer(K, nh, nkv, hd, window):
    """q, k and v as strided views of one projection output, the way the mixer calls it
    (this is the shape of call that the tensor-core kernel takes)."""
    dtype = torch.bfloat16
    news = [200, 1, 64, 65, 333]
    M = sum(news)
    width = (nh + 2 * nkv) * hd
    qkv = randn(M, width, seed=26).to(dtype)
    g = dev(qkv)
    q = g[:, : nh * hd].view(M, nh, hd)
    k = g[:, nh * hd: (nh + nkv) * hd].view(M, nkv, hd)
    v = g[:, (nh + nkv) * hd:].view(M, nkv, hd)
    batch = make_batch("start", list(range(len(news))), [0] * len(news), news)
    scale = 1.0 / math.sqrt(hd)
    from toyinfer_b200.kernels import attention
    for mma_sync in (False, True):          # the tcgen05 kernel, then the mma.sync kernel it replaced
        attention.prefer_mma_sync = mma_sync
        try:
            got = K.attention_prefill(q, k, v, scale, window, batch).cpu().double()
        finally:
            attention.prefer_mma_sync = False
        K.check_status()
        o = 0
        for n in news:
            want = plain_attention_seq(q[o:o + n].cpu(), k[o:o + n].cpu(), v[o:o + n].cpu(), scale, window, dtype)
            torch.testing.assert_close(got[o:o + n], want, **ATT_TOL[dtype])
            o += n


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,window", [(5, 1, 48, 40), (8, 2, 128, 0), (4, 4, 64, 0), (6, 2, 128, 100), (2, 1, 64, 64)])
def test_attention_prefill_beside_rows_of_nan(K, dtype, nh, nkv, hd, window):
    """A sequence's result does not depend on what stands in the rows of other sequences, nor in rows
    that are nobody's (the spare rows of a step of fixed size): those hold NaN here, and a key tile's
    or a query tile's rows reach into them."""
    news = [70, 100, 1, 33, 200, 64, 2]
    bad = (1, 3, 5)
    spare = 59
    M = sum(news)
    total = M + spare
    q = randn(total, nh, hd, seed=27).to(dtype)
    k = randn(total, nkv, hd, seed=28).to(dtype)
    v = randn(total, nkv, hd, seed=29).to(dtype)
    o = 0
    for i, n in enumerate(news):
        if i in bad:
            for t in (q, k, v):
                t[o:o + n] = float("nan")
        o += n
    for t in (q, k, v):
        t[M:] = float("nan")
    batch = make_batch("start", list(range(len(news))), [0] * len(news), news, spare_rows=spare)
    scale = 1.0 / math.sqrt(hd)
    from toyinfer_b200.kernels import attention
    for mma_sync in (False, True):
        attention.prefer_mma_sync = mma_sync
        try:
            got = K.attention_prefill(dev(q), dev(k), dev(v), scale, window, batch).cpu().double()
        finally:
            attention.prefer_mma_sync = False
        K.check_status()
        o = 0
        for i, n in enumerate(news):
            if i not in bad:
                want = plain_attention_seq(q[o:o + n], k[o:o + n], v[o:o + n], scale, window, dtype)
                torch.testing.assert_close(got[o:o + n], want, **ATT_TOL[dtype], msg=lambda m: f"sequence {i}: {m}")
            o += n


@pytest.mark.parametrize("dtype", DT)
def test_attention_prefill_far_key_and_window_edge(K, dtype):
    """One key far back is made to dominate: without a window every later query must
    return its value; with a window only the queries that still see it."""
    nh, nkv, hd, n, far, W = 4, 2, 64, 300, 17, 64
    q = randn(n, nh, hd, seed=23, scale=0.1)
    k = randn(n, nkv, hd, seed=24, scale=0.1)
    v = randn(n, nkv, hd, seed=25)
    k[far] = 0
    k[far, :, 0] = 40.0
    q[:, :, 0] = 40.0            # score with the far key ~ 1600 * scale, others ~ 0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    batch = make_batch("start", [0], [0], [n])
    scale = 1.0 / math.sqrt(hd)
    for window in (0, W):
        got = K.attention_prefill(dev(q), dev(k), dev(v), scale, window, batch).cpu().double()
        want = plain_attention_seq(q, k, v, scale, window, dtype)
        torch.testing.assert_close(got, want, **ATT_TOL[dtype])
        sees = [i for i in range(n) if i >= far and (window == 0 or far > i - window)]
        for i in (sees[0], sees[-1]):
            torch.testing.assert_close(got[i, 0], v[far, 0].double(), rtol=1e-2, atol=1e-2)
        if window:
            first_blind = far + window      # the key at p - window is just outside
            assert (got[first_blind, 0] - v[far, 0].double()).abs().max() > 0.1


def plain_attention_on_gpu(q, k, v, scale, window, dtype):
    """The plain function with its float64 operations on the GPU: for sequences of thousands of
    positions, where the CPU would take minutes."""
    return plain.attention(q.double().cuda(), k.double().cuda(), v.double().cuda(), scale, window, rnd_mode(dtype)).cpu()


@pytest.mark.parametrize("news,window,nh,nkv", [([2048], 0, 4, 2), ([1025, 4097], 0, 4, 2), ([3000, 70], 1000, 4, 2),
                                                ([1300, 600, 129], 0, 32, 8), ([1300, 600, 129], 0, 4, 1), ([257], 0, 2, 1)])
@pytest.mark.parametrize("hd", [128, 64])
def test_attention_prefill_tcgen05_at_long_lengths(K, news, window, nh, nkv, hd):
    """The tcgen05 kernel (head sizes 128 and 64) at the lengths prompts have in practice: 16 to 65
    key tiles per query tile, lengths one past a tile's end, several sequences in one launch; with 32
    heads and three sequences there are more blocks than the device holds at once, so that blocks
    start beside blocks in every stage of their work."""
    dtype = torch.bfloat16
    M = sum(news)
    qkv = randn(M, (nh + 2 * nkv) * hd, seed=27).to(dtype)
    g = dev(qkv)
    q = g[:, : nh * hd].view(M, nh, hd)
    k = g[:, nh * hd: (nh + nkv) * hd].view(M, nkv, hd)
    v = g[:, (nh + nkv) * hd:].view(M, nkv, hd)
    batch = make_batch("start", list(range(len(news))), [0] * len(news), news)
    scale = 1.0 / math.sqrt(hd)
    got = K.attention_prefill(q, k, v, scale, window, batch).cpu().double()
    K.check_status()
    o = 0
    for n in news:
        want = plain_attention_on_gpu(q[o:o + n], k[o:o + n], v[o:o + n], scale, window, dtype)
        torch.testing.assert_close(got[o:o + n], want, **ATT_TOL[dtype])
        o += n


@pytest.mark.parametrize("n,far", [(300, 17), (300, 290), (2048, 5), (2048, 2000), (2048, 1029)])
def test_attention_prefill_tcgen05_far_key(K, n, far):
    """Head size 128 (the tcgen05 kernel, which rescales its output only when a row's maximum has
    grown by more than 2^8): one key dominates, early in the row (the maximum is set in the first
    tile and never moves) or late (every row that sees it has accumulated many tiles at a maximum
    near 0 and must rescale by far more than 2^8 at once).  A second key, between the crowd and the
    dominating one, sits before it and dominates the rows between them, so that the late case
    rescales twice."""
    dtype, nh, nkv, hd = torch.bfloat16, 4, 2, 128
    q = randn(n, nh, hd, seed=123, scale=0.1)
    k = randn(n, nkv, hd, seed=124, scale=0.1)
    v = randn(n, nkv, hd, seed=125)
    k[far] = 0
    k[far, :, 0] = 40.0
    mid = far // 2
    k[mid] = 0
    k[mid, :, 0] = 6.0           # score 240 * scale: about 21 above the crowd, about 2^30 in weight
    q[:, :, 0] = 40.0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    batch = make_batch("start", [0], [0], [n])
    scale = 1.0 / math.sqrt(hd)
    got = K.attention_prefill(dev(q), dev(k), dev(v), scale, 0, batch).cpu().double()
    K.check_status()
    want = plain_attention_on_gpu(q, k, v, scale, 0, dtype)
    torch.testing.assert_close(got, want, **ATT_TOL[dtype])
    for i in (far, n - 1):
        torch.testing.assert_close(got[i, 0], v[far, 0].double(), rtol=1e-2, atol=1e-2)
    if mid > 0 and far - 1 > mid:
        torch.testing.assert_close(got[far - 1, 0], v[mid, 0].double(), rtol=0.05, atol=0.05)


def fill_cache(mem, slot, pages, k, v):
    """k, v [n, kv_heads, hd] into the given pages of a slot (ring-aware)."""
    from toyinfer_b200.cache.manager import PAGE
    n = k.shape[0]
    for i, p in enumerate(pages):
        mem.page_table[slot, i] = p
    for pos in range(n):
        row = pos % mem.ring_rows if mem.ring_rows else pos
        if mem.ring_rows and pos < n - mem.ring_rows:
            continue
        page = pages[row // PAGE]
        mem.k_pages[page, :, row % PAGE] = k[pos]
        mem.v_pages[page, :, row % PAGE] = v[pos]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (5, 1, 48, 40), (8, 4, 64, 0), (8, 2, 128, 0), (4, 4, 128, 64),
                                               (6, 2, 64, 100), (2, 1, 256, 0), (8, 1, 128, 100), (6, 3, 128, 300)])
def test_attention_chunk(K, dtype, nh, nkv, hd, window):
    """New tokens after positions in the cache: (positions held, new tokens) per sequence covers a
    sequence that starts, single tokens, a start in the middle and at the end of a page, runs of
    new tokens longer than a window's ring, and a ring that has wrapped.  Cache lines that no
    query may read hold NaN; so do the lines where this step's own tokens will go."""
    cases = [(0, 70), (64, 1), (65, 40), (300, 1), (129, 130), (1, 1), (200, 200), (127, 2), (700, 300)]
    mem = make_mem(dtype, len(cases), nkv, hd, pages=64, window=window, dirty=float("nan"))
    free = list(range(64, 0, -1))
    scale = 1.0 / math.sqrt(hd)
    ks = [randn(st + n, nkv, hd, seed=130 + i).to(dtype) for i, (st, n) in enumerate(cases)]
    vs = [randn(st + n, nkv, hd, seed=140 + i).to(dtype) for i, (st, n) in enumerate(cases)]
    qs = [randn(st + n, nh, hd, seed=150 + i).to(dtype) for i, (st, n) in enumerate(cases)]
    for s, (st, n) in enumerate(cases):
        total = st + n
        need = (min(total, mem.ring_rows) if mem.ring_rows else total) + 63 >> 6
        pages = [free.pop() for _ in range(need)]
        if st:
            fill_cache(mem, s, pages, dev(ks[s][:st]), dev(vs[s][:st]))
        else:
            for i, pg in enumerate(pages):
                mem.page_table[s, i] = pg
    batch = make_batch("mixed", list(range(len(cases))), [st for st, _ in cases], [n for _, n in cases])
    q = torch.cat([qs[s][st:] for s, (st, _) in enumerate(cases)])
    k = torch.cat([ks[s][st:] for s, (st, _) in enumerate(cases)])
    v = torch.cat([vs[s][st:] for s, (st, _) in enumerate(cases)])
    # one sequence's new rows are NaN as well: its neighbours' tiles reach into them
    bad = 2
    o_bad = sum(n for _, n in cases[:bad])
    for t in (q, k, v):
        t[o_bad:o_bad + cases[bad][1]] = float("nan")
    from toyinfer_b200.kernels import attention
    for mma_sync in (False, True):          # heads of 64 and 128: the tcgen05 kernel, then the mma.sync kernel
        attention.prefer_mma_sync = mma_sync
        try:
            got = K.attention_chunk(dev(q), dev(k), dev(v), mem, scale, window, batch).cpu().double()
        finally:
            attention.prefer_mma_sync = False
        K.check_status()
        o = 0
        for s, (st, n) in enumerate(cases):
            if s != bad:
                want = plain_attention_seq(qs[s], ks[s], vs[s], scale, window, dtype)[st:]
                torch.testing.assert_close(got[o:o + n], want, **ATT_TOL[dtype], msg=lambda m: f"sequence {s} {cases[s]}: {m}")
            o += n


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("hd", [64, 128])
def test_attention_chunk_far_key_in_the_cache(K, dtype, hd):
    """One key far back in the cache dominates every new token's scores; with a window only the
    new tokens that still see it return its value."""
    nh, nkv, st, n, far, W = 4, 2, 500, 90, 449, 128
    k = randn(st + n, nkv, hd, seed=160, scale=0.1)
    v = randn(st + n, nkv, hd, seed=161)
    q = randn(st + n, nh, hd, seed=162, scale=0.1)
    k[far] = 0
    k[far, :, 3] = 40.0
    q[:, :, 3] = 40.0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scale = 1.0 / math.sqrt(hd)
    for window in (0, W):
        mem = make_mem(dtype, 1, nkv, hd, pages=12, window=window, dirty=float("nan"))
        fill_cache(mem, 0, list(range(1, 11)), dev(k[:st]), dev(v[:st]))
        batch = make_batch("mixed", [0], [st], [n])
        got = K.attention_chunk(dev(q[st:]), dev(k[st:]), dev(v[st:]), mem, scale, window, batch).cpu().double()
        want = plain_attention_seq(q, k, v, scale, window, dtype)[st:]
        torch.testing.assert_close(got, want, **ATT_TOL[dtype])
        sees = [i for i in range(n) if window == 0 or far > st + i - window]
        for i in (sees[0], sees[-1]):
            torch.testing.assert_close(got[i, 0], v[far, 0].double(), rtol=1e-2, atol=1e-2)
        if window:
            blind = far + window - st
            assert (got[blind, 0] - v[far, 0].double()).abs().max() > 0.1


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (6, 2, 32, 0), (5, 1, 48, 40), (32, 8, 128, 0),
                                               (8, 1, 128, 100), (2, 2, 256, 0), (16, 1, 64, 0),
                                               (4, 2, 64, 64), (8, 2, 128, 128), (3, 1, 32, 64)])
def test_attention_decode(K, dtype, nh, nkv, hd, window):
    """The last three cases have a window equal to its ring (whole pages, no slack): the newest
    position has overwritten the one that just left the window, and the first and the newest tile
    of a sequence are the same physical page."""
    lens = [1, 64, 65, 300, 129, 100]
    mem = make_mem(dtype, len(lens), nkv, hd, pages=24, window=window, dirty=float("nan"))
    ks = [randn(n, nkv, hd, seed=30 + i).to(dtype) for i, n in enumerate(lens)]
    vs = [randn(n, nkv, hd, seed=40 + i).to(dtype) for i, n in enumerate(lens)]
    free = list(range(24, 0, -1))
    for s, n in enumerate(lens):
        need = (min(n, mem.ring_rows) if mem.ring_rows else n) + 63 >> 6
        fill_cache(mem, s, [free.pop() for _ in range(need)], dev(ks[s]), dev(vs[s]))
    q = randn(len(lens), nh, hd, seed=50).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    from toyinfer_b200.kernels import attention
    # different split counts must agree, and so must the two ways the tensor-core kernel's splits
    # meet: as a cluster through distributed shared memory (chosen when all clusters find room at
    # once) and through global scratch with the combine kernel; each is forced here as well
    for plan, mode in ((64, None), (4096, None), (40960, None), (4096, 1), (40960, 0), (4096, 2), (40960, 2)):
        batch = make_batch("extend", list(range(len(lens))), [n - 1 for n in lens], [1] * len(lens), plan_len=plan)
        attention.force_merge_mode = mode
        try:
            got = K.attention_decode(dev(q), mem, scale, window, batch).cpu().double()
        finally:
            attention.force_merge_mode = None
        K.check_status()
        for s, n in enumerate(lens):
            qq = torch.zeros(n, nh, hd, dtype=dtype)
            qq[-1] = q[s]
            want = plain_attention_seq(qq, ks[s], vs[s], scale, window, dtype)[-1]
            torch.testing.assert_close(got[s], want, **ATT_TOL[dtype])


@pytest.mark.parametrize("nh,nkv,hd,window,norm", [(32, 8, 128, 0, "bf16"), (8, 1, 128, 100, "f32"), (16, 1, 64, 0, "bf16"),
                                                   (40, 8, 128, 0, None), (4, 4, 64, 70, "bf16"),
                                                   (4, 2, 64, 64, "bf16"), (8, 2, 128, 128, "f32")])
@pytest.mark.parametrize("rotate", [True, False])
def test_attention_decode_step_one_kernel_equals_two(K, nh, nkv, hd, window, norm, rotate):
    """The decode kernel with norm, rotation and cache store folded in against the rotate-and-store
    kernel followed by the plain decode kernel: the same output and the same cache, bit for bit
    (both round at the same places).  Lengths at the start, the end and the middle of a page, a
    ring that has wrapped, several split counts, and a layer that borrows its memory (no k, v)."""
    from toyinfer_b200.kernels import attention
    dtype = torch.bfloat16
    lens = [1, 64, 65, 300, 129, 128]
    B = len(lens)
    g = torch.Generator(device="cuda").manual_seed(77)
    mem = make_mem(dtype, B, nkv, hd, pages=30, window=window, dirty=0.0)
    free = list(range(30, 0, -1))
    for s, n in enumerate(lens):
        need = (min(n, mem.ring_rows) if mem.ring_rows else n) + 63 >> 6
        hist_k = torch.randn(n, nkv, hd, generator=g, device="cuda").to(dtype)
        hist_v = torch.randn(n, nkv, hd, generator=g, device="cuda").to(dtype)
        fill_cache(mem, s, [free.pop() for _ in range(need)], hist_k, hist_v)
    qkv = torch.randn(B, (nh + 2 * nkv) * hd + 8, generator=g, device="cuda").to(dtype)      # rows wider than needed: strided views
    wdt = {"bf16": torch.bfloat16, "f32": torch.float32, None: None}[norm]
    q_w = (1 + 0.1 * torch.randn(hd, generator=g, device="cuda")).to(wdt) if wdt else None
    k_w = (1 + 0.1 * torch.randn(hd, generator=g, device="cuda")).to(wdt) if wdt else None
    pos = torch.arange(400, device="cuda", dtype=torch.float32)[:, None] * torch.exp(
        -torch.arange(hd // 2, device="cuda", dtype=torch.float32) / (hd // 2) * math.log(1e4))[None, :]
    tables = (torch.cos(pos).contiguous(), torch.sin(pos).contiguous(), hd) if rotate else None
    scale = 1.0 / math.sqrt(hd)

    def views(buf):
        q = buf[:, :nh * hd].view(B, nh, hd)
        k = buf[:, nh * hd:(nh + nkv) * hd].view(B, nkv, hd)
        v = buf[:, (nh + nkv) * hd:(nh + 2 * nkv) * hd].view(B, nkv, hd)
        return q, k, v

    for plan in (64, 4096):
        for borrow in (False, True):
            batch = make_batch("extend", list(range(B)), [n - 1 for n in lens], [1] * B, plan_len=plan)
            mem_a = type(mem)(mem.k_pages.clone(), mem.v_pages.clone(), mem.page_table, nkv, hd, window, mem.ring_rows)
            mem_b = type(mem)(mem.k_pages.clone(), mem.v_pages.clone(), mem.page_table, nkv, hd, window, mem.ring_rows)
            qa, ka, va = views(qkv.clone())
            qb, kb, vb = views(qkv.clone())
            if borrow:
                ka = va = kb = vb = None
            assert attention.decode_fused_eligible(qb, kb, vb, q_w, k_w, tables, mem_b)
            K.qk_norm_rope_store(qa, ka, va, q_w, k_w, 1e-6, tables, batch, None if borrow else mem_a)
            want = K.attention_decode(qa, mem_a, scale, window, batch)
            before = K.launch_count
            got = K.attention_decode_step(qb, kb, vb, q_w, k_w, 1e-6, tables, mem_b, scale, window, batch)
            assert K.launch_count - before <= 2
            K.check_status()
            assert torch.equal(got, want), (plan, borrow)
            assert torch.equal(mem_a.k_pages, mem_b.k_pages) and torch.equal(mem_a.v_pages, mem_b.v_pages)
            if not borrow:
                assert not torch.equal(mem_b.k_pages, mem.k_pages)      # something was stored


@pytest.mark.parametrize("fused", [False, True])
def test_attention_decode_tensor_cores_at_long_lengths(K, fused):
    """The tensor-core decode kernel (and its form with norm, rotation and store folded in)
    against the plain implementation at the lengths of real contexts: page tables over a hundred
    entries wide, up to 64 live splits and their combine, a batch of very unequal lengths.  The
    plans of 8,192 and 40,960 positions give different split counts for the same data."""
    from toyinfer_b200.parts.rope import rotary_tables
    dtype, nh, nkv, hd, eps = torch.bfloat16, 8, 2, 128, 1e-6
    lens = [8192, 64, 1, 3000, 2048, 4100]
    B = len(lens)
    n_pages = sum((n + 63) // 64 for n in lens)
    mem = make_mem(dtype, B, nkv, hd, pages=n_pages, dirty=float("nan"))
    free = list(range(n_pages, 0, -1))
    ks = [randn(n, nkv, hd, seed=230 + i).to(dtype) for i, n in enumerate(lens)]
    vs = [randn(n, nkv, hd, seed=240 + i).to(dtype) for i, n in enumerate(lens)]
    q = randn(B, nh, hd, seed=250).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    r = rnd_mode(dtype)
    want = []
    if fused:
        # the cache holds all positions but the newest; the step brings that one unformed
        q_w = (1 + randn(hd, seed=251, scale=0.1)).to(dtype)
        k_w = (1 + randn(hd, seed=252, scale=0.1)).to(dtype)
        cos, sin = rotary_tables(hd, 1e6, 8192)
        for s, n in enumerate(lens):
            ang = plain.rope_angles(hd, 1e6, [n - 1])
            qn = plain.rope(plain.rms_norm(q[s:s + 1].double(), q_w, eps, r), ang, r)
            kn = plain.rope(plain.rms_norm(ks[s][n - 1:n].double(), k_w, eps, r), ang, r)
            kk = torch.cat([ks[s][:n - 1].double(), kn])
            qq = torch.zeros(n, nh, hd, dtype=torch.float64)
            qq[-1] = qn[0]
            want.append(plain_attention_on_gpu(qq, kk, vs[s], scale, 0, dtype)[-1])
    else:
        for s, n in enumerate(lens):
            qq = torch.zeros(n, nh, hd, dtype=dtype)
            qq[-1] = q[s]
            want.append(plain_attention_on_gpu(qq, ks[s], vs[s], scale, 0, dtype)[-1])
    for s, n in enumerate(lens):
        held = n - 1 if fused else n
        pages = [free.pop() for _ in range((n + 63) // 64)]
        if held:
            fill_cache(mem, s, pages, dev(ks[s][:held]), dev(vs[s][:held]))
        else:
            mem.page_table[s, 0] = pages[0]
    k_clean, v_clean = mem.k_pages.clone(), mem.v_pages.clone()
    for plan in (8192, 40960):
        mem.k_pages.copy_(k_clean)
        mem.v_pages.copy_(v_clean)
        batch = make_batch("extend", list(range(B)), [n - 1 for n in lens], [1] * B, plan_len=plan)
        if fused:
            k_new = torch.stack([ks[s][n - 1] for s, n in enumerate(lens)])
            v_new = torch.stack([vs[s][n - 1] for s, n in enumerate(lens)])
            got = K.attention_decode_step(dev(q).clone(), dev(k_new), dev(v_new), dev(q_w), dev(k_w), eps,
                                          (dev(cos), dev(sin), hd), mem, scale, 0, batch).cpu().double()
        else:
            got = K.attention_decode(dev(q), mem, scale, 0, batch).cpu().double()
        K.check_status()
        for s in range(B):
            torch.testing.assert_close(got[s], want[s], **ATT_TOL[dtype], msg=lambda m: f"plan {plan}, length {lens[s]}: {m}")


@pytest.mark.parametrize("dtype", DT)
def test_attention_decode_far_key(K, dtype):
    nh, nkv, hd, n, far = 8, 2, 64, 700, 3
    k = randn(n, nkv, hd, seed=60, scale=0.1)
    v = randn(n, nkv, hd, seed=61)
    k[far] = 0
    k[far, :, 1] = 30.0
    q = randn(1, nh, hd, seed=62, scale=0.1)
    q[:, :, 1] = 30.0
    k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
    mem = make_mem(dtype, 1, nkv, hd, pages=12)
    fill_cache(mem, 0, list(range(12, 0, -1))[:11], dev(k), dev(v))
    batch = make_batch("extend", [0], [n - 1], [1])
    got = K.attention_decode(dev(q), mem, 1.0 / math.sqrt(hd), 0, batch).cpu().double()
    for h in range(nh):
        torch.testing.assert_close(got[0, h], v[far, h // 4].double(), rtol=1e-2, atol=1e-2)


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("V", [256, 1000, 151936])
def test_argmax(K, V):
    x = randn(5, V, seed=70)
    x[1, 17] = x[1, 900 % V] = 50.0          # a tie: the lower index wins
    got = K.argmax(dev(x)).cpu().tolist()
    assert got == [plain.argmax(r) for r in x]


def test_argmax_ties_across_blocks_and_odd_rows(K):
    """A row is scanned by several blocks: equal maxima far apart, zeros of both signs, NaNs,
    a row of -inf, rows that start off a 16-byte boundary, many rows (one block each), and
    the same call again (the kernel leaves its scratch as it found it)."""
    V = 151936
    x = randn(6, V, seed=71) - 100.0
    x[0, 140000] = x[0, 3] = 7.0                       # tie: first and last block
    x[1, :] = -1.0
    x[1, 99999], x[1, 12345] = 0.0, -0.0               # -0 at the lower index equals +0: it wins
    x[2, 5] = float("nan")
    x[2, 77777] = 3.0
    x[3, :] = float("-inf")                            # first index of the maximum: 0
    x[4, V - 1] = 9.0
    x[5, :] = float("nan")
    want = [3, 12345, 77777, 0, V - 1, 0]
    xd = dev(x)
    for _ in range(3):
        assert K.argmax(xd).cpu().tolist() == want
    odd = torch.zeros(6, V + 3, device="cuda")
    odd[:, 1:V + 1] = xd
    assert K.argmax(odd[:, 1:V + 1]).cpu().tolist() == want
    many = randn(700, 333, seed=72)
    assert K.argmax(dev(many)).cpu().tolist() == [plain.argmax(r) for r in many]
    assert K.argmax(xd[:1]).cpu().tolist() == want[:1]


@pytest.mark.parametrize("V,top_k,top_p,temp", [(300, 0, 1.0, 0.8), (300, 20, 0.95, 0.6), (5000, 50, 0.5, 1.3),
                                                (151936, 20, 0.95, 0.6), (1000, 1000, 1.0, 0.7),
                                                (2000, 1024, 0.9, 1.0)])
@pytest.mark.parametrize("two_kernels", [True, False])
def test_sample_matches_plain(K, monkeypatch, V, top_k, top_p, temp, two_kernels):
    """``two_kernels``: the usual settings (top_k up to 64; temperature alone) as two short kernels over
    many blocks, or every setting in its one-block-per-row form."""
    monkeypatch.setattr(K, "two_kernel_sampling", two_kernels)
    R = 6
    x = randn(R, V, seed=71, scale=3.0)
    x[2, 5] = x[2, 9] = x[2].max() + 1      # tied maxima
    keys = torch.arange(100, 100 + R, dtype=torch.int64)
    steps = torch.arange(R, dtype=torch.int32)
    got = K.sample(dev(x), temp, top_k if top_k < V else 0, top_p, 1234, dev(keys), dev(steps)).cpu().tolist()
    for r in range(R):
        u = plain.uniform_from(1234, int(keys[r]), int(steps[r]))
        assert abs(u - K.uniform_from(1234, int(keys[r]), int(steps[r]))) == 0.0
        want = plain.sample(x[r], temp, top_k, top_p, u)
        if got[r] != want:
            # allowed only when the draw falls within float rounding of a boundary between
            # the two tokens' cumulative intervals
            alt = {plain.sample(x[r], temp, top_k, top_p, min(max(u + d, 0.0), 0.99999994)) for d in (-3e-6, 3e-6)}
            assert got[r] in alt, (r, got[r], want, alt)


@pytest.mark.parametrize("V,top_k,top_p,temp", [(151936, 20, 0.95, 0.6), (151936, 64, 1.0, 1.0), (5000, 50, 0.5, 1.3), (4097, 1, 1.0, 0.7),
                                                (300, 40, 0.9, 0.8), (9000, 33, 0.999, 2.0), (151936, 1000, 0.9, 1.0), (2000, 1024, 0.95, 0.7),
                                                (151936, 200, 1.0, 0.8)])
def test_sample_top_k_in_two_kernels_gives_the_one_kernel_picks(K, monkeypatch, V, top_k, top_p, temp):
    """With top_k up to 1,024 the two-kernel form keeps the same entries in the same order and then does
    the one-kernel form's arithmetic: the same token, draw by draw, also where many entries are equal
    (quantised logits: the lowest indices among the equal ones are kept) and where the k-th value is
    shared by entries of different chunks."""
    R = 32
    x = randn(R, V, seed=75, scale=3.0)
    x[1] = torch.round(x[1] * 2) / 2                    # many equal values
    x[2] = torch.round(x[2])
    x[3, ::4096 // 3] = x[3].max() + 0.5                # the largest value many times, in several chunks
    x[4] = 0.0                                          # all equal: the first top_k indices are kept
    x[4, 1::2] = -0.0
    keys = torch.arange(500, 500 + R, dtype=torch.int64)
    picks = {}
    for two in (True, False):
        monkeypatch.setattr(K, "two_kernel_sampling", two)
        picks[two] = [K.sample(dev(x), temp, top_k, top_p, 99, dev(keys), dev(torch.full((R,), st, dtype=torch.int32))).cpu().tolist()
                      for st in range(6)]
    assert picks[True] == picks[False]
    assert all(p < top_k for st in picks[True] for p in [st[4]])      # row 4: only the first top_k indices can be drawn


def exact_picks(x, temp, top_k, top_p, u, slack):
    """The sampling rule (plain.sample's) in float64, vectorised, for every combination of u and
    top_p moved by -slack, 0, +slack: the set of tokens between the lowest and the highest rank
    picked.  Two float32 implementations that add up thousands of probabilities in different
    orders are each within rounding of the exact running sum, but not of each other's token when the
    draw falls next to a boundary; `slack` is that rounding expressed in units of the running sum."""
    xs = x.double() / temp
    V = xs.numel()
    neg, order = torch.sort(-xs, stable=True)          # larger first, lower index first among equals
    k = top_k if 0 < top_k < V else V
    p = torch.exp(-neg[:k] - (-neg[0]))
    cum = torch.cumsum(p / p.sum(), 0)
    ranks = []
    for tp in (top_p - slack, top_p, top_p + slack):
        over = (cum > tp).nonzero()
        n = int(over[0]) + 1 if len(over) else k
        for uu in (u - slack, u, u + slack):
            coin = min(max(uu, 0.0), 1.0) * cum[n - 1]
            hit = (cum[:n] > coin).nonzero()
            ranks.append(int(hit[0]) if len(hit) else n - 1)
    return set(order[min(ranks):max(ranks) + 1].tolist()), k


@pytest.mark.parametrize("V,top_k,top_p,temp,scale,quantum", [
    (300, 0, 0.9, 0.8, 3.0, 0),            # a nucleus over the whole (small) vocabulary
    (5000, 0, 0.5, 1.3, 3.0, 0),           # the cut falls in the first tier of 1,024
    (5000, 3000, 0.97, 1.0, 3.0, 0),       # more candidates than one sort holds: three tiers
    (2000, 1500, 1.0, 0.7, 3.0, 0),        # top_k above 1,024 without top_p
    (20000, 0, 0.9, 5.0, 3.0, 0),          # a flat distribution: the nucleus spans a dozen tiers
    (6000, 0, 0.9, 2.0, 3.0, 0.5),         # values on a grid of 0.5: ties everywhere, also across tier boundaries
    (6000, 2500, 0.8, 2.0, 3.0, 1.0),
])
@pytest.mark.parametrize("two_kernels", [True, False])
def test_sample_any_top_k_and_top_p(K, monkeypatch, V, top_k, top_p, temp, scale, quantum, two_kernels):
    """The settings beyond one shared-memory sort (top_p without top_k, top_k above 1,024), draw by
    draw: the token is the plain (float32) sampler's, or the exact rule's for a draw within the
    rounding of a float32 running sum over the kept entries (4 standard deviations of a random walk
    of n roundings of 2^-25 each).  ``two_kernels``: top_p without top_k first looks for the nucleus
    among the row's 64 largest entries (found by many blocks) and leaves the row to the tiered kernel
    only where it is larger; else the tiered kernel does every row."""
    monkeypatch.setattr(K, "two_kernel_sampling", two_kernels)
    R = 4
    x = randn(R, V, seed=73, scale=scale)
    if quantum:
        x = torch.round(x / quantum) * quantum
    keys = torch.arange(200, 200 + R, dtype=torch.int64)
    steps = torch.arange(3, 3 + R, dtype=torch.int32)
    for seed in (1234, 99):
        got = K.sample(dev(x), temp, top_k, top_p, seed, dev(keys), dev(steps)).cpu().tolist()
        for r in range(R):
            u = plain.uniform_from(seed, int(keys[r]), int(steps[r]))
            if got[r] == plain.sample(x[r], temp, top_k, top_p, u):
                continue
            n = top_k if 0 < top_k < V else V
            allowed, _ = exact_picks(x[r], temp, top_k, top_p, u, 4 * math.sqrt(n) * 2.0 ** -25)
            assert got[r] in allowed, (seed, r, got[r], allowed)


@pytest.mark.parametrize("two_kernels", [True, False])
def test_sample_nucleus_over_a_large_vocabulary(K, monkeypatch, two_kernels):
    """top_k off and top_p 0.95 at the vocabulary of the benchmark model: a peaked row (the nucleus is
    a handful of tokens: drawn by the kernel that looks among the 64 largest, when that form is on)
    and a flat one (tens of tiers)."""
    monkeypatch.setattr(K, "two_kernel_sampling", two_kernels)
    V = 151936
    x = randn(2, V, seed=74, scale=1.5)
    x[0, 777] = 14.0
    x[0, 90000] = 13.0
    keys = torch.tensor([5, 6], dtype=torch.int64)
    steps = torch.tensor([0, 9], dtype=torch.int32)
    got = K.sample(dev(x), 0.6, 0, 0.95, 7, dev(keys), dev(steps)).cpu().tolist()
    for r in range(2):
        u = plain.uniform_from(7, int(keys[r]), int(steps[r]))
        allowed, _ = exact_picks(x[r], 0.6, 0, 0.95, u, 4 * math.sqrt(V) * 2.0 ** -25)
        assert got[r] in allowed, (r, got[r], allowed)
    assert got[0] in (777, 90000)


def test_sample_distribution(K):
    """Many draws from a small distribution land where softmax(logits / T) says."""
    V, n = 8, 20000
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -2.0, 3.0, 0.2])
    x = logits.repeat(n, 1)
    keys = torch.arange(n, dtype=torch.int64)
    steps = torch.zeros(n, dtype=torch.int32)
    got = K.sample(dev(x), 0.7, 0, 1.0, 99, dev(keys), dev(steps)).cpu()
    freq = torch.bincount(got.long(), minlength=V).double() / n
    p = torch.softmax(logits.double() / 0.7, 0)
    assert (freq - p).abs().max() < 0.015


# ---------------------------------------------------------------------------
def test_a_wait_that_runs_out_is_reported_and_leaves_the_library_usable(K):
    """Every device-side wait of the library is bounded; a wait that runs out records a code in the
    status word and the kernel returns.  Here the library's test kernel waits, with a limit of
    10,000 polls, on a barrier nothing arrives on: it must come back, check_status() must raise with
    the code of a wait for a load, the scratch that kernels share (tickets) must be clear again even
    if something had left a ticket set, the next product must be right, and the word must be clear."""
    from toyinfer_b200.kernels import KernelError, gemm
    K.check_status()
    x = randn(40, 512, seed=300).to(torch.bfloat16)
    w = randn(2560, 512, seed=301, scale=0.05).to(torch.bfloat16)
    want = x.double() @ w.double().T
    K.linear(dev(x), dev(w))                            # makes sure the ticket array exists
    tickets = gemm._tickets_for(torch.device("cuda", torch.cuda.current_device()))
    tickets[3] = 1                                      # as a product that gave up half-way would leave it
    assert K.testing_wait_runs_out(10000) is True
    with pytest.raises(KernelError, match="status 1: a wait for a TMA load ran out"):
        K.check_status()
    assert int(tickets.abs().sum()) == 0
    got = K.linear(dev(x), dev(w)).cpu().double()
    torch.testing.assert_close(got, want, rtol=1.6e-2, atol=2e-2)
    K.check_status()                                    # clear: no second report


@pytest.mark.parametrize("dtype", DT)
def test_embed_scale_and_logit_scale_cap(K, dtype):
    V, H, M = 50, 72, 9
    table = randn(V, H, seed=310).to(dtype)
    ids = torch.randint(0, V, (M,), generator=torch.Generator().manual_seed(311), dtype=torch.int32)
    got = K.embed(dev(table), dev(ids), 8.5).cpu().double()
    want = plain.rnd(table[ids.long()].double() * 8.5, rnd_mode(dtype))
    torch.testing.assert_close(got, want, **tol(dtype))
    logits = randn(5, 1003, seed=312, scale=20.0)
    buf = torch.full((5, 1100), 7.0)
    buf[:, :1003] = logits
    g = dev(buf)
    out = K.logit_scale_cap(g[:, :1003], 0.25, 30.0)
    want = 30.0 * torch.tanh(logits.double() * 0.25 / 30.0)
    torch.testing.assert_close(out.cpu().double(), want, rtol=2e-6, atol=2e-6)
    assert torch.all(g[:, 1003:].cpu() == 7.0)          # the rows' tails are untouched
    out = K.logit_scale_cap(dev(logits).clone(), 2.0, 0.0)
    torch.testing.assert_close(out.cpu(), logits * 2.0, rtol=0, atol=0)


def test_kernels_give_the_same_bits_every_time(K):
    """Races show as results that change from launch to launch.  The kernels whose blocks hand work
    to one another (tensor-core attention with its pipelines, products whose tiles are shared or
    split, decode attention with split keys) run a dozen times each on a device-filling case, and
    every run must give the first run's bits."""
    dtype = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(77)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)

    cases = []
    nh, nkv, hd = 32, 8, 128
    news = [1300, 600, 129]
    M = sum(news)
    qkv = rnd(M, (nh + 2 * nkv) * hd)
    q, k, v = qkv[:, :nh * hd].view(M, nh, hd), qkv[:, nh * hd:(nh + nkv) * hd].view(M, nkv, hd), qkv[:, (nh + nkv) * hd:].view(M, nkv, hd)
    batch = make_batch("start", [0, 1, 2], [0, 0, 0], news)
    cases.append(("prompt attention", lambda: K.attention_prefill(q, k, v, 1 / math.sqrt(hd), 0, batch)))
    q64, k64, v64 = q.view(M, 2 * nh, 64), k.view(M, 2 * nkv, 64), v.view(M, 2 * nkv, 64)      # the same rows as heads of 64
    cases.append(("prompt attention, heads of 64", lambda: K.attention_prefill(q64, k64, v64, 0.125, 0, batch)))
    # new tokens after cached positions
    starts = [700, 64, 1000]
    mem = make_mem(dtype, 3, nkv, hd, pages=80)
    free = list(range(80, 0, -1))
    for s, (st, n) in enumerate(zip(starts, news)):
        pages = [free.pop() for _ in range((st + n + 63) // 64)]
        fill_cache(mem, s, pages, rnd(st, nkv, hd), rnd(st, nkv, hd))
    mixed = make_batch("mixed", [0, 1, 2], starts, news)
    cases.append(("chunk attention", lambda: K.attention_chunk(q, k, v, mem, 1 / math.sqrt(hd), 0, mixed)))
    # decode attention with split keys, eight sequences
    lens = [2000, 1999, 64, 65, 1500, 700, 1, 1024]
    dmem = make_mem(dtype, 8, nkv, hd, pages=160)
    free = list(range(160, 0, -1))
    for s, n in enumerate(lens):
        fill_cache(dmem, s, [free.pop() for _ in range((n + 63) // 64)], rnd(n, nkv, hd), rnd(n, nkv, hd))
    dq = rnd(8, nh, hd)
    dbatch = make_batch("extend", list(range(8)), [n - 1 for n in lens], [1] * 8, plan_len=2048)
    cases.append(("decode attention", lambda: K.attention_decode(dq, dmem, 1 / math.sqrt(hd), 0, dbatch)))
    for Mx, N, Kd in ((4096, 2560, 4096), (2048, 2560, 4096), (1300, 3600, 264), (64, 2560, 9728), (8, 2560, 9728), (2048, 6144, 2560)):
        x, w = rnd(Mx, Kd), rnd(N, Kd, scale=0.03)
        cases.append((f"product {Mx} x {N} x {Kd}", lambda x=x, w=w: K.linear(x, w)))
    for what, fn in cases:
        first = fn().clone()
        for i in range(12):
            again = fn()
            assert torch.equal(first, again), f"{what}: run {i + 2} differs from the first"
        K.check_status()

"""The order in which the many-token matrix product deals out its tiles, checked on the host: the
library's own walk (the code the kernels run, compiled for the host too) is traced for many shapes
and the properties the kernels rely on are checked.  Needs nvcc to build the library, no GPU."""
from __future__ import annotations

import ctypes
import random
import shutil

import pytest

pytestmark = pytest.mark.skipif(shutil.which("nvcc") is None, reason="the kernel library cannot be built without nvcc")


def _trace(M, N, K, sms):
    from toyinfer_b200.kernels.lib import library
    lib = library()
    cap = 1 << 16
    rows = (ctypes.c_int * (cap * 8))()
    units, tiles, pair = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    fn = lib.ti_gemm_walk_trace
    fn.restype = ctypes.c_int
    n = fn(M, N, K, sms, rows, cap, ctypes.byref(units), ctypes.byref(tiles), ctypes.byref(pair))
    assert n <= cap
    out = [tuple(rows[i * 8:(i + 1) * 8]) for i in range(n)]
    return out, units.value, tiles.value, bool(pair.value)


def _check(M, N, K, sms):
    rows, units, tiles, pair = _trace(M, N, K, sms)
    if not rows:
        return None
    nkb = (K + 63) // 64
    covered = {}
    per_tile = {}
    per_unit = {}
    for unit, tile, kb0, kb1, whole, place, other, other_place in rows:
        assert 0 <= unit < units and 0 <= tile < tiles and 0 <= kb0 < kb1 <= nkb
        assert bool(whole) == (kb0 == 0 and kb1 == nkb)
        for kb in range(kb0, kb1):
            assert (tile, kb) not in covered, "a step of the contraction is done twice"
            covered[(tile, kb)] = unit
        per_tile.setdefault(tile, []).append((unit, kb0, kb1, place, other, other_place))
        per_unit.setdefault(unit, []).append((tile, kb0, kb1, whole, place))
    assert len(covered) == tiles * nkb, "a step of the contraction is left out"
    shared = 0
    for tile, pieces in per_tile.items():
        if len(pieces) == 1:
            continue
        shared += 1
        assert len(pieces) == 2, "a tile in more than two pieces"
        (ua, a0, a1, pa, oa, opa), (ub, b0, b1, pb, ob, opb) = sorted(pieces, key=lambda p: p[1])
        assert a0 == 0 and a1 == b0 and b1 == nkb                # the pieces meet
        assert ub == ua + 1                                      # neighbours in the cut
        assert (oa, opa) == (ub, pb) and (ob, opb) == (ua, pa)   # each finds the other's piece where it was put
    for unit, pieces in per_unit.items():
        places = [(p[4]) for p in pieces if not p[3]]
        assert len(places) <= 2 and len(set(places)) == len(places), "two pieces of a unit in one place"
    # work is even: no unit has more than a step over its share of the shared tiles, plus whole rounds
    steps = [sum(k1 - k0 for _, k0, k1, _, _ in per_unit.get(u, [])) for u in range(units)]
    assert max(steps) - min(steps) <= nkb
    return shared, pair


@pytest.mark.parametrize("M,N,K", [(2048, 2560, 4096), (2048, 2560, 9728), (2048, 6144, 2560), (2048, 19456, 2560),
                                   (1300, 3600, 264), (16384, 19456, 2560), (8192, 12288, 4096), (512, 19456, 264),
                                   (1100, 3000, 328), (777, 3000, 328), (2048, 151936, 2560), (4741, 520, 264)])
def test_every_step_once_and_pieces_meet(M, N, K):
    _check(M, N, K, 148)


def test_tiles_for_a_round_and_a_bit():
    """2,048 x 2,560 outputs are 80 tiles of 256 x 256 for 74 pairs: they run as 72 tiles of 256 x 288 in one
    round (whole tiles, nothing shared); 4,096 tokens x 2,560 (2.2 rounds) and a one-SM shape are shared out."""
    shared, pair = _check(2048, 2560, 4096, 148)
    assert pair and shared == 0
    assert _plan(2048, 2560, 4096, 148)[1] == 288 and _plan(2048, 4096, 12288, 148)[1] == 512
    shared, pair = _check(4096, 2560, 4096, 148)
    assert pair and shared > 0
    shared, pair = _check(1300, 3600, 264, 148)
    assert not pair and shared > 0


def _plan(M, N, K, sms):
    from toyinfer_b200.kernels.lib import library
    swap, bn, splits, tickets, ws = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_longlong()
    library().ti_linear_tc_plan(M, N, K, sms, ctypes.byref(swap), ctypes.byref(bn), ctypes.byref(splits), ctypes.byref(ws),
                                ctypes.byref(tickets))
    return bool(swap.value), bn.value, splits.value, ws.value, tickets.value


@pytest.mark.parametrize("sms", [148, 132, 37])
def test_the_plan_asks_for_the_workspace_and_tickets_the_walk_uses(sms):
    rng = random.Random(11)
    for _ in range(200):
        M = rng.choice([1, 8, 16, 33, 64, 65, 300, 512, 1300, 2048, 5000])
        N = rng.choice([128, 520, 2560, 3600, 6144, 19456])
        K = rng.choice([64, 264, 2560, 4096, 9728])
        swap, bn, splits, ws, tickets = _plan(M, N, K, sms)
        assert bn % 16 == 0 and 16 <= bn <= 512 and splits >= 1
        rows, units, tiles, pair = _trace(M, N, K, sms)
        if splits > 1:
            assert not rows                                   # a split contraction runs one block per tile
            rows_a, rows_b = (N, M) if swap else (M, N)
            n_tiles = -(-rows_a // 128) * -(-rows_b // bn)
            assert ws == splits * n_tiles * 128 * bn and tickets == n_tiles
            continue
        pieces = [r for r in rows if not r[4]]
        if not pieces:          # whole tiles only (also when the cuts fall on tile borders, as with one step per tile)
            continue
        blocks = 2 if pair else 1
        assert units * blocks <= sms
        # a place for every piece: (unit, place, block of the unit), a tile's rows of one block in each
        assert ws >= units * 2 * blocks * 128 * bn
        assert tickets >= (max(r[1] for r in pieces) + 1) * blocks


def test_random_shapes_and_device_sizes():
    rng = random.Random(7)
    walked = 0
    for _ in range(300):
        sms = rng.choice([148, 132, 108, 64, 37, 2, 1])
        M = rng.choice([65, 129, 300, 512, 640, 1000, 2048, 3000, 5000, 9000])
        N = rng.choice([256, 520, 1000, 2560, 3600, 6144, 12288, 19456])
        K = rng.choice([64, 72, 264, 1000, 2560, 4096, 9728])
        if _check(M, N, K, sms) is not None:
            walked += 1
    assert walked > 100


def test_row_groups_of_the_few_token_product_fill_the_places_and_never_overflow_them():
    """The few-token product's weight rows per group (8 to 16, even when gated): whenever groups of 16 rows
    fit the places that the SMs offer at once, the groups are the smallest (down to 8 rows) that still fit."""
    from toyinfer_b200.kernels.lib import library
    fn = library().ti_skinny_rows_per_group
    fn.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_int]
    fn.restype = ctypes.c_int
    assert fn(2560, 296, 0) == 9 and fn(6144, 444, 0) == 14 and fn(19456, 444, 1) == 16 and fn(2560, 296, 1) == 10
    rng = random.Random(3)
    for _ in range(3000):
        places = rng.choice([1, 2, 60, 148, 264, 296, 444, 592, 1184])
        n = rng.randint(1, 20 * places + 40)
        for gated in (0, 1):
            rows = fn(n, places, gated)
            assert 8 <= rows <= 16 and (not gated or rows % 2 == 0)
            groups = -(-n // rows)
            if -(-n // 16) > places:
                assert rows == 16                       # more than one round anyway: whole groups
            else:
                assert groups <= places
                smaller = rows - (2 if gated else 1)
                if smaller >= 8:
                    assert -(-n // smaller) > places    # the next smaller group would overflow the places

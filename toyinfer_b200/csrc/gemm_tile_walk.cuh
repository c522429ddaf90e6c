// The order in which the units of the many-token matrix product take their work: plain
// arithmetic on tile and step numbers, for the kernels (gemm_tcgen05_walk.cuh) and for the host
// (a trace of it for tests: ti_gemm_walk_trace in gemm_tcgen05.cu).
#pragma once

namespace tigemm {
// What a unit does, in order.  The tiles seldom fill whole rounds of units (2,048 x 2,560
// outputs are 160 tiles of 128 x 256 for 148 SMs: two rounds, the second nearly empty).  So the
// first `shared` tiles, between one and two rounds' worth, are not dealt out tile by tile but as
// one row of shared * nkb contraction steps cut into equal parts, one per unit: a unit finishes
// the tile its part starts in, takes whole tiles, and begins the tile its part ends in.  A part
// is at least a tile long, so a tile has two pieces at most.  Pieces go to a float32 workspace
// (two places per block: the piece at the start of its part and the one at its end), and the
// block that brings a tile's second piece (a ticket per tile and block of the unit) adds the two
// and stores the tile.  The remaining tiles follow in whole rounds.
struct Piece {
    int tile, kb0, kb1;
    bool whole;     // the whole contraction: stored straight from tensor memory
    int place;      // else: which of the block's two places in the workspace takes it
};
struct TileWalk {
    int nkb, n_tiles, next_whole, stride;
    long long at, end;
    bool first;
    __host__ __device__ TileWalk(int shared, int n_tiles_, int nkb_, int unit, int units) : nkb(nkb_), n_tiles(n_tiles_), first(true) {
        const long long steps = (long long)shared * nkb_;
        at = part_start(unit, steps, units);
        end = part_start(unit + 1, steps, units);
        next_whole = shared + unit;
        stride = units;
    }
    __host__ __device__ static long long part_start(int unit, long long steps, int units) { return (long long)unit * steps / units; }
    __host__ __device__ bool next(Piece& p) {
        if (at < end) {
            p.tile = (int)(at / nkb);
            p.kb0 = (int)(at - (long long)p.tile * nkb);
            const long long left = end - at;
            const int len = left < nkb - p.kb0 ? (int)left : nkb - p.kb0;
            p.kb1 = p.kb0 + len;
            p.whole = len == nkb;
            p.place = first ? 0 : 1;
            first = false;
            at += len;
            return true;
        }
        if (next_whole < n_tiles) {
            p.tile = next_whole; p.kb0 = 0; p.kb1 = nkb; p.whole = true; p.place = 0;
            next_whole += stride;
            return true;
        }
        return false;
    }
    // the unit whose part holds contraction step `s` of the shared tiles
    __host__ __device__ static int unit_of(long long s, long long steps, int units) {
        int u = (int)(s * units / steps);
        while (u + 1 < units && part_start(u + 1, steps, units) <= s) u++;
        while (u > 0 && part_start(u, steps, units) > s) u--;
        return u;
    }
    // For the unit that holds a piece of a shared tile: the unit that holds the other piece, and
    // which of that unit's two places in the workspace the piece lies in (0: the first piece of
    // its part, which begins inside this tile; 1: its last, its part began before).
    __host__ __device__ static void other_piece(int tile, int nkb, int unit, long long steps, int units, int& other, int& place) {
        const long long t0 = (long long)tile * nkb;
        const int u0 = unit_of(t0, steps, units);
        other = u0 == unit ? u0 + 1 : u0;
        place = part_start(other, steps, units) >= t0 ? 0 : 1;
    }
};
}  // namespace tigemm

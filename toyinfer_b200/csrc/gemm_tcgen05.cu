// out = X W^T in bfloat16 on the 5th-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands staged in shared memory by TMA.
//
// The kernel computes D[i, j] = sum_k A[i, k] B[j, k] for a tile of 128 rows of A and BN
// rows of B, both operands K-contiguous ("K-major"), which is how activations [tokens, K]
// and weights [out, K] already lie in memory.  Either may play A:
//   * many tokens (prefill): A = activations, B = weights, D stored as out[i, j];
//   * few tokens (decode):   A = weights, B = activations (BN = 16..64), D stored
//     transposed as out[j, i].  The weight matrix is streamed once at full width of the
//     128-row MMA whatever the batch; the step is bound by that read.
// The contraction may be split over blockIdx.z; partial tiles go to a float32 workspace and
// the last block to finish a tile (a ticket per tile) adds them in split order, so the
// result does not depend on timing.  The many-token kernel (every SM walking over tiles, alone
// or as one of a pair on the two-SM MMA, cta_group::2) shares out the tiles of an uneven last
// round by contraction steps instead: TileWalk.
//
// Roles inside a block of 192 threads: warp 0 issues TMA loads into a ring of stages
// (full/empty mbarriers), one lane of warp 1 issues the MMAs (four K = 16 steps per
// 64-wide stage) and commits them to the stage's empty barrier, warps 2..5 read the
// accumulator back with tcgen05.ld (each its own 32 TMEM lanes) and store.  Every wait is
// bounded (see tma.cuh); a block always frees its tensor memory before it returns.
//
// Contraction and rounding are those of the reference's projections (src/decode.cu:202-236,
// src/prefill.cu:124-161): bfloat16 operands, float32 accumulation, one rounding of the result.
#include "gemm_tcgen05.cuh"
#include "gemm_tile_walk.cuh"

#include <map>
#include <mutex>
#include <tuple>

using namespace tigemm;

namespace {
// ---- host ------------------------------------------------------------------
struct MapKey {
    const void* ptr; long long rows, cols, stride; int box_rows;
    bool operator<(const MapKey& o) const {
        return std::tie(ptr, rows, cols, stride, box_rows) < std::tie(o.ptr, o.rows, o.cols, o.stride, o.box_rows);
    }
};
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_lock;

int operand_map(const void* ptr, long long rows, long long cols, long long stride_elems, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_lock);
    MapKey key{ptr, rows, cols, stride_elems, box_rows};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        CUtensorMap m;
        if (int rc = ti_make_tensor_map_2d_bf16(&m, ptr, (uint64_t)rows, (uint64_t)cols, (uint64_t)stride_elems * 2,
                                                (uint32_t)box_rows, BK))
            return rc;
        if (g_maps.size() > 8192) g_maps.clear();
        it = g_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

// How many tiles of a many-token product are shared out by contraction steps (TileWalk): with
// whole rounds of tiles, or less than one round, none; else the last round and the one before it,
// so that every unit's part is at least a tile long.
int shared_tiles_of(int tiles, int units) {
    if (units <= 0 || tiles < units || tiles % units == 0) return 0;
    return units + tiles % units;
}

// Weight rows per tile for many tokens.  Wider tiles are a little more efficient per flop; what
// counts besides is how much of the last tile along the weights' rows is used, and, where the
// tiles are dealt out whole (`whole_rounds`), how well they fill whole rounds of `sms` blocks.
int wide_tile(int rows_a, int rows_b, int sms, bool whole_rounds, double* score_out = nullptr) {
    const int cand[9] = {256, 240, 224, 208, 192, 176, 160, 144, 128};
    const double mma_eff[9] = {1.0, 0.99, 0.98, 0.97, 0.96, 0.95, 0.94, 0.92, 0.90};
    int best = 256;
    double best_score = -1.0;
    for (int c = 0; c < 9; c++) {
        const int tiles = ((rows_a + BM - 1) / BM) * ((rows_b + cand[c] - 1) / cand[c]);
        const int rounds = (tiles + sms - 1) / sms;
        const double useful = (double)rows_b / (((rows_b + cand[c] - 1) / cand[c]) * (double)cand[c]);
        double score = mma_eff[c] * useful;
        if (whole_rounds) score *= tiles / ((double)rounds * sms);
        if (score > best_score + 1e-9) { best_score = score; best = cand[c]; }
    }
    if (score_out) *score_out = best_score;
    return best;
}
}  // namespace

// For tests and measurements: 0 lets the plan choose, 1 keeps many-token products on one SM per
// tile, 2 puts them on two wherever there are enough tiles.
static int g_pair_mode = 0;
extern "C" void ti_set_gemm_pair_mode(int mode) { g_pair_mode = mode; }
// For measurements: with bn > 0, products of more than 64 tokens that do not run on pairs take tiles
// of bn weight rows and split the contraction `splits` ways (0: as planned).
static int g_force_bn = 0, g_force_splits = 0;
extern "C" void ti_set_gemm_force(int bn, int splits) { g_force_bn = bn; g_force_splits = splits; }


namespace {
struct Plan {
    bool swap;          // few tokens: the weights are the MMA's row operand
    int bn;             // rows of the other operand per tile
    int splits;         // of the contraction, over blockIdx.z (the one-tile-per-block kernel)
    bool walk;          // the many-token kernel
    bool pair;          // ... on two SMs per tile
    int shared;         // ... tiles shared out by contraction steps
    int tiles;
    long long ws_floats;
    int tickets;
};

Plan make_plan(int M, int N, int K, int sms) {
    Plan p = {};
    p.swap = M <= 64;
    const int rows_a = p.swap ? N : M, rows_b = p.swap ? M : N;
    const int nkb = (K + BK - 1) / BK;
    int b;
    bool share = false;     // many tokens: tiles shared out by contraction steps
    if (p.swap) {
        b = rows_b <= 16 ? 16 : rows_b <= 32 ? 32 : 64;
        // A matrix with few row tiles is split along the contraction, and the block that adds a
        // tile's partial sums does so in rounds whose number grows with the tile's width.  While
        // the blocks still fit the SMs once, such a product takes its tokens in two tiles of half
        // the width (measured at 64 tokens: 2560 x 4096 16.5 -> 12.1 us, 6144 x 2560 14.9 -> 13.0,
        // 2560 x 9728 21.2 -> 18.5; at 32 tokens 2560 x 4096 11.7 -> 9.9); the weights' second
        // reader finds them in L2.
        const int row_tiles = (rows_a + BM - 1) / BM;
        if (b == 64 && row_tiles * 2 <= sms) b = 32;
        else if (b == 32 && rows_b > 16 && row_tiles * 4 <= sms) b = 16;
    }
    else if (rows_b >= 256) {
        // Two SMs per tile of 256 x 256 where that wastes little at the edges and there is at least
        // a tile per pair; what the rounds leave over is shared out by contraction steps.
        const int pairs = sms / 2;
        const long long tiles_a2 = (rows_a + 2 * BM - 1) / (2 * BM), tiles_b2 = (rows_b + 255) / 256;
        const double useful = ((double)rows_a / (tiles_a2 * 2 * BM)) * ((double)rows_b / (tiles_b2 * 256));
        // A product whose tiles of 256 x 256 are between one and two rounds of pairs takes wider
        // tiles that fit one round where such a width exists: all pairs then walk the contraction in
        // step (see gemm_tcgen05_walk.cuh).  Measured at 2,048 tokens, shared out by steps against one
        // round of wide tiles: 4,096 x 12,288 (512 wide) 201 -> 138 us, 4,096 x 4,096 53 -> 50;
        // 3,072 tokens x 2,560 x 9,728 133 -> 108; 2,048 x 2,560 x 9,728 (288 wide: two MMAs of 144
        // columns) 87.0 -> 85.3, x 4,096 41.7 -> 40.4.
        int fit = 0;
        if (g_pair_mode != 1 && pairs > 0 && tiles_a2 <= pairs && tiles_a2 * tiles_b2 > pairs && tiles_a2 * tiles_b2 < 2 * pairs &&
            ((double)rows_a / (tiles_a2 * 2 * BM) >= 0.93 || (rows_a + BM - 1) / BM == 2 * tiles_a2)) {
            // (the tokens fill their tiles of 256, as for any pair, or tiles of 128 would hold as many empty rows:
            // 192 tokens x 19,456 x 2,560 35.3 -> 27 us)
            const int cols = (int)(pairs / tiles_a2);                       // column tiles of one round
            const int need = (rows_b + cols - 1) / cols;                    // weight rows each must hold
            const int widths[4] = {288, 320, 384, 512};
            for (int w = 0; w < 4 && !fit; w++)
                if (widths[w] >= need) fit = widths[w];
            // one round of wide tiles against the steps of the shared-out form, which run about 1.3 times slower each
            if (fit && (double)fit / 256.0 > 0.95 * 1.3 * (double)(tiles_a2 * tiles_b2) / pairs) fit = 0;
        }
        if (fit) {
            p.pair = true;
            b = fit;
        }
        else if (g_pair_mode != 1 && pairs > 0 && tiles_a2 * tiles_b2 >= pairs && (useful >= 0.93 || g_pair_mode == 2)) {
            p.pair = true;
            b = 256;
            // Sharing costs about as much as a dozen steps of the contraction (measured at 2,048
            // tokens: 6,144 weight rows x 2,560 gain nothing from it, 19,456 x 2,560 gain 8 %).
            const long long tiles2 = tiles_a2 * tiles_b2;
            const long long idle_steps = ((tiles2 + pairs - 1) / pairs) * nkb - tiles2 * nkb / pairs;
            share = idle_steps > 20;
        } else {
            // The width that fills whole rounds best.  Where even that leaves more than a tenth of the
            // device idle (measured at 2,048 tokens: 2,560 weight rows do, 6,144 and 19,456 do not), the
            // widest useful tile instead, with a part of the tiles shared out by contraction steps.
            double score;
            b = wide_tile(rows_a, rows_b, sms, true, &score);
            if (score < 0.89) {
                const int wide = wide_tile(rows_a, rows_b, sms, false);
                if (((rows_a + BM - 1) / BM) * ((rows_b + wide - 1) / wide) >= sms) { b = wide; share = true; }
            }
        }
    }
    else b = rows_b > 64 ? 128 : rows_b > 32 ? 64 : rows_b > 16 ? 32 : 16;
    if (g_force_bn > 0 && !p.swap && !p.pair) { b = g_force_bn; share = false; }
    const int tile_rows = p.pair ? 2 * BM : BM;
    const int tiles = ((rows_a + tile_rows - 1) / tile_rows) * ((rows_b + b - 1) / b);
    int sp = 1;
    // measured with the weights as the row operand (16, 32, 64 tokens, the four products of a 4B-shaped
    // layer): 1.5 blocks per SM are 2-4 % faster in sum than 1.0, 2.0 are 10 % slower
    const int want = p.swap ? sms + sms / 2 : sms;
    if (tiles < want && !p.pair) {
        if (p.swap) {
            sp = (want + tiles / 2) / tiles;
            if (sp < 1) sp = 1;
            const int max_sp = nkb / 4 > 0 ? nkb / 4 : 1;       // at least four 64-wide blocks per split
            if (sp > max_sp) sp = max_sp;
            if (sp > 32) sp = 32;
        } else {
            // 65 to some hundred tokens: a block is alone on its SM, so the blocks must fit the SMs in
            // one round; a block that adds up a tile reads each 64 KB piece through its one SM, and a
            // part of the contraction shorter than 20 steps is not worth its ramp.  Measured (us, 4B
            // shapes, splits as rounded before -> so): 256 tokens x 6,144 x 2,560 25.4 -> 15.0 (two
            // rounds of 192 blocks -> 96 whole tiles), x 2,560 x 4,096 23.2 -> 16.9, x 2,560 x 9,728
            // 33.7 -> 24.5 (160 blocks -> 120); 512 x 2,560 x 4,096 29.8 -> 20.0, x 9,728 50.7 -> 41.1;
            // 128 x 2,560 x 4,096 19.2 -> 16.6 (7 splits -> 3), x 9,728 23.9 -> 21.6 (7 -> 4).
            sp = sms / tiles;
            if (sp > nkb / 20) sp = nkb / 20;
            if (sp > 4) sp = 4;
            if (sp < 1) sp = 1;
        }
        // drop splits that would get no work
        const int per = (nkb + sp - 1) / sp;
        sp = (nkb + per - 1) / per;
    }
    if (g_force_bn > 0 && g_force_splits > 0 && !p.swap && !p.pair) {
        const int per = (nkb + g_force_splits - 1) / g_force_splits;
        sp = (nkb + per - 1) / per;
    }
    p.bn = b; p.splits = sp; p.tiles = tiles;
    p.ws_floats = sp > 1 ? (long long)sp * tiles * BM * b : 0;
    p.tickets = sp > 1 ? tiles : 0;
    p.walk = !p.swap && sp == 1 && b >= 128;
    if (p.walk) {
        // two places per block for the pieces of shared tiles, a ticket per shared tile and block of a unit
        p.shared = share ? shared_tiles_of(tiles, p.pair ? sms / 2 : sms) : 0;
        p.ws_floats = p.shared ? (long long)sms * 2 * BM * b : 0;
        p.tickets = p.shared * (p.pair ? 2 : 1);
    }
    return p;
}
}  // namespace

// Floats of workspace and tickets (`n_tiles`) ti_linear_tc needs for this shape (0: none), and
// how it splits.  `sms` blocks fill the device once.
extern "C" int ti_linear_tc_plan(int M, int N, int K, int sms, int* swap, int* bn, int* splits, long long* ws_floats,
                                 int* n_tiles) {
    const Plan p = make_plan(M, N, K, sms);
    *swap = p.swap; *bn = p.bn; *splits = p.splits; *ws_floats = p.ws_floats; *n_tiles = p.tickets;
    return 0;
}

// x[M, K] (row stride ldx), w[N, K] (row stride ldw), both bfloat16; out[M, N] bfloat16 or
// float32 with row stride ldo.  With `gated`, w's rows are (gate_0, up_0, gate_1, up_1, ...) and
// out is [M, N / 2] = up * gate / (1 + exp(-gate)).  `workspace` (float32) and `tickets` (int32, zero before the
// first use, left zero) as planned by ti_linear_tc_plan; tickets needs n_tiles entries and may be
// null, in which case a second kernel adds the partial tiles of a split contraction, and the
// many-token kernel deals out whole tiles only.
extern "C" int ti_linear_tc(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                            long long ldw, long long ldo, int out_f32, int gated, int sms, float* workspace, int* tickets,
                            cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    TI_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    TI_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "linear (tcgen05): K and the row strides must be multiples of 8 elements");
    TI_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "linear (tcgen05): operands must be 16-byte aligned");
    const Plan p = make_plan(M, N, K, sms);
    const int swap = p.swap, bn = p.bn, splits = p.splits;
    TI_REQUIRE(splits == 1 || workspace, "linear (tcgen05): a split contraction needs a workspace");
    GemmArgs g;
    g.rows_a = swap ? N : M; g.rows_b = swap ? M : N; g.K = K;
    g.out = out; g.ld_out = ldo; g.out_f32 = out_f32; g.transposed = swap;
    g.splits = splits; g.workspace = workspace; g.tickets = tickets;
    g.gated = gated;
    g.shared_tiles = p.walk && workspace && tickets ? p.shared : 0;      // without them: whole tiles only
    TI_REQUIRE(!gated || (N % 2 == 0 && !out_f32), "linear (tcgen05): a gated product needs an even number of weight rows and a bfloat16 result");
    CUtensorMap am, bm;
    if (int rc = operand_map(swap ? w : x, g.rows_a, K, swap ? ldw : ldx, BM, &am)) return rc;
    // the other operand's box: a whole tile's rows; a pair's block loads half of them, or, where the
    // tile takes two MMAs per step, a quarter at a time
    if (int rc = operand_map(swap ? x : w, g.rows_b, K, swap ? ldx : ldw, p.pair ? (bn > 256 ? bn / 4 : bn / 2) : bn, &bm)) return rc;
    if (p.pair) return launch_walk_pair(bn, am, bm, g, sms, stream);
    if (p.walk) return launch_walk_single(bn, am, bm, g, sms, stream);
    return launch_tile(bn, am, bm, g, stream);
}

// For tests: what every unit of a many-token product of this shape does, as the kernel will walk
// it.  Rows of 8 ints: unit, tile, first step, end step, whole tile (0/1), place of the piece, and
// for a piece of a shared tile the unit and place of the other piece as the adding block works
// them out (else -1).  Returns the number of rows (at most max_rows are written); *units_out and
// *tiles_out receive the number of units and tiles, *pair_out whether two SMs take a tile.
extern "C" int ti_gemm_walk_trace(int M, int N, int K, int sms, int* rows, int max_rows, int* units_out, int* tiles_out,
                                  int* pair_out) {
    const Plan p = make_plan(M, N, K, sms);
    *pair_out = p.pair ? 1 : 0;
    *tiles_out = p.tiles;
    *units_out = 0;
    if (!p.walk) return 0;
    const int all_units = p.pair ? sms / 2 : sms;
    const int units = p.shared > 0 || p.tiles > all_units ? all_units : p.tiles;
    const int nkb = (K + BK - 1) / BK;
    *units_out = units;
    int n = 0;
    for (int u = 0; u < units; u++) {
        TileWalk walk(p.shared, p.tiles, nkb, u, units);
        Piece piece;
        while (walk.next(piece)) {
            if (n < max_rows) {
                int* r = rows + (size_t)n * 8;
                r[0] = u; r[1] = piece.tile; r[2] = piece.kb0; r[3] = piece.kb1; r[4] = piece.whole ? 1 : 0; r[5] = piece.place;
                r[6] = r[7] = -1;
                if (!piece.whole) TileWalk::other_piece(piece.tile, nkb, u, (long long)p.shared * nkb, units, r[6], r[7]);
            }
            n++;
        }
    }
    return n;
}

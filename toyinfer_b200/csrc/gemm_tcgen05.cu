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
#include "tcgen05.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace {
constexpr int BM = 128, BK = 64, THREADS = 192;

struct GemmArgs {
    int rows_a, rows_b, K;
    void* out; long long ld_out; int out_f32; int transposed;
    int splits; float* workspace; int* tickets;
    int gated;      // rows of the weight operand come in (gate, up) pairs: store up * silu(gate), half as many columns
    int shared_tiles;   // many-token kernel: the first so many tiles are shared out by contraction steps (see TileWalk)
};

// kind::f16 instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, M = 128
template <int BN>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Narrow tiles (few tokens, the weights stream) keep five stages so that two blocks share an
// SM: a grid of about one block per SM then leaves room for the next kernel's blocks, which
// request their weights while this kernel is still running.  Wide tiles take the SM alone.
template <int BN> constexpr int stages_for() {
    constexpr int per = BM * BK * 2 + BN * BK * 2;
    constexpr int n = (200 * 1024) / per;
    return BN <= 32 ? 5 : BN == 64 ? 4 : (n > 8 ? 8 : n);
}
template <int BN> constexpr int blocks_per_sm() { return BN <= 64 ? 2 : 1; }

// Stores 16 consecutive columns (c .. c+15 of the tile that starts at column b0) of row i of D.
// All lanes of a warp must call it together (the gated, transposed form exchanges values
// between neighbouring lanes).
__device__ __forceinline__ void store_chunk(const GemmArgs& g, int i, int b0, int c, float (&r)[16], int lane) {
    if (g.gated) {
        // gate and up are neighbours along the weight operand's rows; both are rounded to
        // the storage type first, as if the product had been stored (src/decode.cu:756-762)
        if (g.transposed) {
            // neighbours are lanes 2n and 2n+1: the even lane stores column i / 2
#pragma unroll
            for (int e = 0; e < 16; e++) {
                const float mine = __bfloat162float(__float2bfloat16_rn(r[e]));
                const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                const int j = b0 + c + e;
                if ((lane & 1) == 0 && i < g.rows_a && j < g.rows_b)
                    ((bf16*)g.out)[(size_t)j * g.ld_out + (i >> 1)] =
                        __float2bfloat16_rn(other * (mine / (1.0f + expf(-mine))));
            }
        } else if (i < g.rows_a) {
            const int j0 = b0 + c;
            bf16* o = (bf16*)g.out + (size_t)i * g.ld_out + (j0 >> 1);
            uint32_t pk[4];
            float z[8];
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float gate = __bfloat162float(__float2bfloat16_rn(r[2 * e]));
                const float up = __bfloat162float(__float2bfloat16_rn(r[2 * e + 1]));
                z[e] = up * (gate / (1.0f + expf(-gate)));
            }
            if (j0 + 16 <= g.rows_b && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(z[2 * e], z[2 * e + 1]);
                    pk[e] = *reinterpret_cast<uint32_t*>(&v);
                }
                *reinterpret_cast<uint4*>(o) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; e++) if (j0 + 2 * e + 1 < g.rows_b) o[e] = __float2bfloat16_rn(z[e]);
            }
        }
    } else if (i < g.rows_a) {
        if (g.transposed) {
            // out[j, i]: the warp's lanes are consecutive i, so each j is one coalesced store
#pragma unroll
            for (int e = 0; e < 16; e++) {
                const int j = b0 + c + e;
                if (j < g.rows_b) {
                    if (g.out_f32) ((float*)g.out)[(size_t)j * g.ld_out + i] = r[e];
                    else ((bf16*)g.out)[(size_t)j * g.ld_out + i] = __float2bfloat16_rn(r[e]);
                }
            }
        } else {
            const int j0 = b0 + c;
            if (g.out_f32) {
                float* o = (float*)g.out + (size_t)i * g.ld_out + j0;
                if (j0 + 16 <= g.rows_b && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
                    for (int e = 0; e < 16; e += 4) *reinterpret_cast<float4*>(o + e) = make_float4(r[e], r[e + 1], r[e + 2], r[e + 3]);
                } else {
#pragma unroll
                    for (int e = 0; e < 16; e++) if (j0 + e < g.rows_b) o[e] = r[e];
                }
            } else {
                bf16* o = (bf16*)g.out + (size_t)i * g.ld_out + j0;
                if (j0 + 16 <= g.rows_b && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
                    uint32_t pk[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        __nv_bfloat162 v = __floats2bfloat162_rn(r[2 * e], r[2 * e + 1]);
                        pk[e] = *reinterpret_cast<uint32_t*>(&v);
                    }
                    *reinterpret_cast<uint4*>(o) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4*>(o + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                } else {
#pragma unroll
                    for (int e = 0; e < 16; e++) if (j0 + e < g.rows_b) o[e] = __float2bfloat16_rn(r[e]);
                }
            }
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(THREADS, blocks_per_sm<BN>())
gemm_tc_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
               GemmArgs g, int* status) {
    ti_pdl_trigger();
    constexpr int STAGES = stages_for<BN>();
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr uint32_t TMEM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[STAGES], empty[STAGES], acc_ready;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_last, s_gave_up;

    // Once a wait has run out somewhere, results are lost anyway: later blocks leave at once
    // instead of each running into its own limits.
    if (threadIdx.x == 0) s_gave_up = *reinterpret_cast<volatile int*>(status);
    __syncthreads();
    if (s_gave_up) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * BM, b0 = blockIdx.y * BN, split = blockIdx.z;
    const int nkb = (g.K + BK - 1) / BK;
    const int per = (nkb + g.splits - 1) / g.splits;
    const int kb0 = split * per, kb1 = min(nkb, kb0 + per);
    const int n_iter = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(&acc_ready, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        __syncwarp();
        tmem_alloc(&tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    // The weights are constant, so their tiles for the first stages are requested now, while
    // the kernel before this one may still be running; only the activations have to wait.
    const int n_pre = min(STAGES, n_iter);
    const bool weights_are_a = g.transposed != 0;
    if (warp == 0 && lane == 0) {
        for (int it = 0; it < n_pre; it++) {
            unsigned char* sa = smem + (size_t)it * (A_BYTES + B_BYTES);
            mbar_expect_tx(&full[it], A_BYTES + B_BYTES);
            if (weights_are_a) tma_load_2d(sa, &a_map, (kb0 + it) * BK, a0, &full[it]);
            else tma_load_2d(sa + A_BYTES, &b_map, (kb0 + it) * BK, b0, &full[it]);
        }
    }
    ti_pdl_sync();      // from here on memory written by earlier kernels may be read

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            for (int it = 0; it < n_pre; it++) {
                unsigned char* sa = smem + (size_t)it * (A_BYTES + B_BYTES);
                if (weights_are_a) tma_load_2d(sa + A_BYTES, &b_map, (kb0 + it) * BK, b0, &full[it]);
                else tma_load_2d(sa, &a_map, (kb0 + it) * BK, a0, &full[it]);
            }
            for (int it = n_pre; it < n_iter; it++) {
                const int s = it % STAGES;
                if (!mbar_wait(&empty[s], (uint32_t)(((it / STAGES) & 1) ^ 1))) { ti_report(status, TI_STATUS_PIPE_WAIT); break; }
                unsigned char* sa = smem + (size_t)s * (A_BYTES + B_BYTES);
                mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                tma_load_2d(sa, &a_map, (kb0 + it) * BK, a0, &full[s]);
                tma_load_2d(sa + A_BYTES, &b_map, (kb0 + it) * BK, b0, &full[s]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc<BN>();
            bool ok = true;
            for (int it = 0; it < n_iter && ok; it++) {
                const int s = it % STAGES;
                if (!mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1))) { ti_report(status, TI_STATUS_TMA_WAIT); ok = false; break; }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + (size_t)s * (A_BYTES + B_BYTES));
                const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; k++)   // 16 elements = 32 bytes = 2 descriptor units along K
                    tc_mma_bf16(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (it > 0 || k > 0) ? 1u : 0u);
                tc_commit(&empty[s]);               // the stage is free once these MMAs have read it
            }
            if (ok) tc_commit(&acc_ready);          // the accumulator is complete once all MMAs are done
        }
    } else {
        // ---- epilogue: warps 2..5, each reads the 32 TMEM lanes it may access
        const int q = warp & 3;                     // lanes q*32 .. q*32+31
        const int i = a0 + q * 32 + lane;           // row of A this thread holds
        bool ok = true;
        if (n_iter > 0) {
            if (!mbar_wait(&acc_ready, 0)) { ti_report(status, TI_STATUS_MMA_WAIT); ok = false; }
            ok = __all_sync(0xffffffffu, ok);   // the reads below are warp-wide instructions
            tc_fence_after();
        }
        const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
        if (g.splits > 1) {
            // partial tile to the workspace, element (i, j) at [j * 128 + i_local]
            float* ws = g.workspace + (((size_t)split * gridDim.x + blockIdx.x) * gridDim.y + blockIdx.y) * (size_t)(BM * BN);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float r[16];
                if (ok && n_iter > 0) tmem_ld16(taddr + c, r);
                else {
#pragma unroll
                    for (int e = 0; e < 16; e++) r[e] = 0.f;
                }
#pragma unroll
                for (int e = 0; e < 16; e++) ws[(size_t)(c + e) * BM + q * 32 + lane] = r[e];
            }
            if (!g.tickets) ok = false;             // a second kernel adds the partial tiles
            else {
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) {
                const int tile = blockIdx.x * gridDim.y + blockIdx.y;
                const int prev = atomicAdd(&g.tickets[tile], 1);
                s_last = prev == g.splits - 1;
                if (s_last) g.tickets[tile] = 0;    // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!s_last) ok = false;                // another block finishes this tile
            else __threadfence();
            }
        }
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float r[16];
                if (g.splits > 1) {
                    // partial tiles are added in split order; four splits' loads are in flight together
#pragma unroll
                    for (int e = 0; e < 16; e++) r[e] = 0.f;
                    const size_t tile_off = ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * (size_t)(BM * BN) + (size_t)c * BM + q * 32 + lane;
                    const size_t split_stride = (size_t)gridDim.x * gridDim.y * (size_t)(BM * BN);
                    for (int sp0 = 0; sp0 < g.splits; sp0 += 4) {
                        float t4[4][16];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const bool live = sp0 + u < g.splits;
                            const float* ws = g.workspace + (size_t)(live ? sp0 + u : sp0) * split_stride + tile_off;
#pragma unroll
                            for (int e = 0; e < 16; e++) t4[u][e] = live ? __ldcg(&ws[(size_t)e * BM]) : 0.f;
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++)
#pragma unroll
                            for (int e = 0; e < 16; e++) r[e] += t4[u][e];
                    }
                } else if (n_iter > 0) {
                    tmem_ld16(taddr + c, r);
                } else {
#pragma unroll
                    for (int e = 0; e < 16; e++) r[e] = 0.f;
                }
                store_chunk(g, i, b0, c, r, lane);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// Many tokens: every SM walks over output tiles (activations as the MMA's row operand, BN
// weight rows per tile).  Two accumulators in tensor memory: while the epilogue warps read one
// back and store it, the MMA warp already fills the other, so the tensor cores do not idle
// during a tile's epilogue.  The TMA ring runs on across tile borders.
//
// Two forms.  One block per tile of 128 tokens; or (PAIR) the two blocks of a cluster on one
// tile of 256 tokens with the two-SM MMA (cta_group::2): each loads its 128 tokens and BN / 2 of
// the weight rows, so an SM takes in 32 KB per 64 steps of the contraction where a block on its
// own takes 48 KB for the same arithmetic.  The block of rank 0 issues the MMAs for both; all
// loads of a stage are counted on its `full` barrier; a commit frees the stage, and hands over
// the accumulator, in both blocks at once; the epilogue warps of both report a drained
// accumulator to rank 0.  Each block reads its own 128 rows of the result from its own tensor
// memory.  "Unit" below is what works on a tile: a block, or a pair of them.
// ---------------------------------------------------------------------------
template <int BN, bool PAIR> constexpr int walk_stages() {
    constexpr int per = BM * BK * 2 + (PAIR ? BN / 2 : BN) * BK * 2;
    constexpr int n = (196 * 1024) / per;
    return n > 8 ? 8 : n;
}

// Order of the tiles of a many-token product.  Token tiles go in groups of 2,048 tokens: within a
// group the token tile changes fastest, then the weight tile, so the units that run together
// share few weight tiles and one panel of activations, and the panel (2,048 tokens x K, some
// tens of MB at most) stays in L2 while the group sweeps over all weight tiles.  Without the
// grouping every round of units would touch all token tiles: fine while the activations fit L2
// (2,048 tokens), a re-read of all of them per weight tile when they do not (16,384).
constexpr int PANEL_TOKENS = 2048;
__device__ __forceinline__ void tile_origin(int tile, int tiles_a, int tiles_b, int tile_rows, int bn, int& a0, int& b0) {
    const int panel = PANEL_TOKENS / tile_rows;
    const int per_group = panel * tiles_b;
    const int grp = tile / per_group, within = tile - grp * per_group;
    const int first = grp * panel;
    const int span = min(panel, tiles_a - first);
    a0 = (first + within % span) * tile_rows;
    b0 = (within / span) * bn;
}

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
    __device__ TileWalk(int shared, int n_tiles_, int nkb_, int unit, int units) : nkb(nkb_), n_tiles(n_tiles_), first(true) {
        const long long steps = (long long)shared * nkb_;
        at = part_start(unit, steps, units);
        end = part_start(unit + 1, steps, units);
        next_whole = shared + unit;
        stride = units;
    }
    __device__ static long long part_start(int unit, long long steps, int units) { return (long long)unit * steps / units; }
    __device__ bool next(Piece& p) {
        if (at < end) {
            p.tile = (int)(at / nkb);
            p.kb0 = (int)(at - (long long)p.tile * nkb);
            const int len = (int)min((long long)(nkb - p.kb0), end - at);
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
    __device__ static int unit_of(long long s, long long steps, int units) {
        int u = (int)(s * units / steps);
        while (u + 1 < units && part_start(u + 1, steps, units) <= s) u++;
        while (u > 0 && part_start(u, steps, units) > s) u--;
        return u;
    }
};

template <int BN, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_walk_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                    GemmArgs g, int* status) {
    ti_pdl_trigger();
    constexpr int STAGES = walk_stages<BN, PAIR>();
    constexpr int B_ROWS = PAIR ? BN / 2 : BN;                  // weight rows this block loads
    constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;               // tokens of a tile
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = B_ROWS * BK * 2;
    constexpr uint32_t ACC_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;   // columns of one accumulator
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int s_gave_up, s_last;

    if (!PAIR) {
        // Once a wait has run out somewhere, results are lost anyway (see gemm_tc_kernel).  A pair
        // has no such exit: its blocks must leave together.
        if (threadIdx.x == 0) s_gave_up = *reinterpret_cast<volatile int*>(status);
        __syncthreads();
        if (s_gave_up) return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = PAIR ? (int)cluster_rank() : 0;
    const int unit = PAIR ? blockIdx.x >> 1 : blockIdx.x, units = PAIR ? gridDim.x >> 1 : gridDim.x;
    const int tiles_a = (g.rows_a + TILE_ROWS - 1) / TILE_ROWS, tiles_b = (g.rows_b + BN - 1) / BN;
    const int n_tiles = tiles_a * tiles_b;
    const int nkb = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], PAIR ? 8 : 4); }   // epilogue warps of the unit
        mbar_fence_init();
    }
    if (PAIR) {
        __syncthreads();
        cluster_sync_all();         // the other block's barriers exist before anything arrives on them
    }
    if (warp == 1) {
        __syncwarp();
        if (PAIR) { tmem_alloc_pair(&tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
        else { tmem_alloc(&tmem_slot, TMEM_COLS); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    ti_pdl_sync();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            TileWalk walk(g.shared_tiles, n_tiles, nkb, unit, units);
            Piece p;
            while (ok && walk.next(p)) {
                int a0, b0;
                tile_origin(p.tile, tiles_a, tiles_b, TILE_ROWS, BN, a0, b0);
                a0 += rank * BM;
                b0 += rank * B_ROWS;
                for (int kb = p.kb0; kb < p.kb1; kb++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty[s], (uint32_t)(((it / STAGES) & 1) ^ 1))) { ti_report(status, TI_STATUS_PIPE_WAIT); ok = false; break; }
                    unsigned char* sa = smem + (size_t)s * (A_BYTES + B_BYTES);
                    if (PAIR) {
                        if (rank == 0) mbar_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));
                        const uint32_t bar = cluster_addr(&full[s], 0);
                        tma_load_2d_pair(sa, &a_map, kb * BK, a0, bar);
                        tma_load_2d_pair(sa + A_BYTES, &b_map, kb * BK, b0, bar);
                    } else {
                        mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                        tma_load_2d(sa, &a_map, kb * BK, a0, &full[s]);
                        tma_load_2d(sa + A_BYTES, &b_map, kb * BK, b0, &full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
            int it = 0, n = 0;
            bool ok = true;
            TileWalk walk(g.shared_tiles, n_tiles, nkb, unit, units);
            Piece p;
            for (; ok && walk.next(p); n++) {
                const int buf = n & 1;
                // the epilogue must have drained this accumulator (its use before last)
                if (!mbar_wait(&acc_empty[buf], (uint32_t)(((n >> 1) & 1) ^ 1))) { ti_report(status, TI_STATUS_PIPE_WAIT); ok = false; break; }
                tc_fence_after();
                const uint32_t acc = tmem + buf * ACC_COLS;
                for (int kb = p.kb0; kb < p.kb1; kb++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1))) { ti_report(status, TI_STATUS_TMA_WAIT); ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)s * (A_BYTES + B_BYTES));
                    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        const uint32_t accumulate = (kb > p.kb0 || k > 0) ? 1u : 0u;
                        if (PAIR) tc_mma_bf16_pair(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accumulate);
                        else tc_mma_bf16(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accumulate);
                    }
                    if (PAIR) tc_commit_pair(&empty[s]); else tc_commit(&empty[s]);
                }
                if (ok) { if (PAIR) tc_commit_pair(&acc_full[buf]); else tc_commit(&acc_full[buf]); }
            }
        }
    } else {
        const int q = warp & 3;
        int n = 0;
        bool ok = true;
        TileWalk walk(g.shared_tiles, n_tiles, nkb, unit, units);
        Piece p;
        const long long shared_steps = (long long)g.shared_tiles * nkb;
        constexpr size_t TILE_FLOATS = (size_t)BM * BN;         // of one block's rows of a tile
        const int blocks_per_unit = PAIR ? 2 : 1;
        // this warp has read its lanes of the accumulator: hand it back to the MMA warp
        auto release = [&](int buf) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(cluster_addr(&acc_empty[buf], 0));
                else mbar_arrive(&acc_empty[buf]);
            }
        };
        for (; walk.next(p); n++) {
            const int buf = n & 1;
            int a0, b0;
            tile_origin(p.tile, tiles_a, tiles_b, TILE_ROWS, BN, a0, b0);
            const int i = a0 + rank * BM + q * 32 + lane;
            if (!mbar_wait(&acc_full[buf], (uint32_t)((n >> 1) & 1))) { ti_report(status, TI_STATUS_MMA_WAIT); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem + buf * ACC_COLS + ((uint32_t)(q * 32) << 16);
            if (p.whole) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float r[16];
                    tmem_ld16(taddr + c, r);
                    store_chunk(g, i, b0, c, r, lane);
                }
                release(buf);
                continue;
            }
            // A piece of a tile.  The two units that hold this tile's pieces, by the cut of the steps:
            const long long t0 = (long long)p.tile * nkb;
            const int u0 = TileWalk::unit_of(t0, shared_steps, units);
            const int other = u0 == unit ? u0 + 1 : u0;
            const int t = q * 32 + lane;
            int* ticket = &g.tickets[p.tile * blocks_per_unit + rank];
            // Has the other unit brought its piece already?  Then this block adds the tile up and
            // its own piece never leaves tensor memory.  Else the piece goes to this block's place
            // in the workspace (thread t keeps 16 columns as four float4, word v of chunk c at
            // [(c / 16 * 4 + v) * 128 + t]), and the ticket says whether the other came meanwhile.
            asm volatile("bar.sync 1, 128;" ::: "memory");      // everyone has read s_last of the piece before
            if (threadIdx.x == 64) s_last = *reinterpret_cast<volatile int*>(ticket) == 1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            bool last = s_last != 0;
            if (!last) {
                float4* mine = reinterpret_cast<float4*>(g.workspace + (((size_t)unit * 2 + p.place) * blocks_per_unit + rank) * TILE_FLOATS) + t;
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float r[16];
                    tmem_ld16(taddr + c, r);
#pragma unroll
                    for (int v = 0; v < 4; v++) mine[(size_t)(c / 4 + v) * BM] = make_float4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) s_last = atomicAdd(ticket, 1) == 1;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                last = s_last != 0;
            }
            if (last) {
                if (threadIdx.x == 64) *ticket = 0;             // ready for the next launch
                __threadfence();
                // Nothing runs beside this at the end of a kernel, so the other piece is fetched 128
                // columns at a time, all loads in flight together, before this block's own piece is
                // read back and added (a sum of two, the same whichever block forms it).
                const int place = TileWalk::part_start(other, shared_steps, units) >= t0 ? 0 : 1;   // first piece of its part, or last
                const float4* ws = reinterpret_cast<const float4*>(g.workspace + (((size_t)other * 2 + place) * blocks_per_unit + rank) * TILE_FLOATS) + t;
                constexpr int GROUP = 8;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16 * GROUP) {
                    float4 f[GROUP][4];
#pragma unroll
                    for (int u = 0; u < GROUP; u++)
#pragma unroll
                        for (int v = 0; v < 4; v++)
                            f[u][v] = c0 + 16 * u < BN ? __ldcg(&ws[(size_t)((c0 + 16 * u) / 4 + v) * BM]) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < GROUP; u++) {
                        const int c = c0 + 16 * u;
                        if (c >= BN) break;
                        float r[16];
                        tmem_ld16(taddr + c, r);
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            r[4 * v] += f[u][v].x; r[4 * v + 1] += f[u][v].y; r[4 * v + 2] += f[u][v].z; r[4 * v + 3] += f[u][v].w;
                        }
                        store_chunk(g, i, b0, c, r, lane);
                    }
                }
            }
            release(buf);
        }
    }
    // A block of a pair neither leaves nor gives back its tensor memory while the other may
    // still read its shared memory or arrive on its barriers.
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem, TMEM_COLS); else tmem_dealloc(tmem, TMEM_COLS);
    }
}

// Adds the partial tiles of a split contraction (workspace layout as written above) in split order
// and stores the result; one thread per (row of A, 16 columns).
template <int BN>
__global__ void splitk_reduce_kernel(GemmArgs g, int tiles_a, int tiles_b) {
    ti_pdl_trigger();
    ti_pdl_sync();
    const int lane = threadIdx.x & 31;
    const int chunks = BN / 16;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     // (tile, 32-row group, chunk)
    const long long n_items = (long long)tiles_a * tiles_b * 4 * chunks;
    if (item >= n_items) return;
    const int c = (int)(item % chunks) * 16;
    const int q = (int)((item / chunks) % 4);
    const int tile = (int)(item / (chunks * 4));
    const int ta = tile / tiles_b, tb = tile % tiles_b;
    const int i = ta * BM + q * 32 + lane;
    float r[16];
#pragma unroll
    for (int e = 0; e < 16; e++) r[e] = 0.f;
    for (int sp = 0; sp < g.splits; sp++) {
        const float* ws = g.workspace + (((size_t)sp * tiles_a + ta) * tiles_b + tb) * (size_t)(BM * BN);
#pragma unroll
        for (int e = 0; e < 16; e++) r[e] += ws[(size_t)(c + e) * BM + q * 32 + lane];
    }
    store_chunk(g, i, tb * BN, c, r, lane);
}

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

template <int BN>
int launch(const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, cudaStream_t stream) {
    constexpr int STAGES = stages_for<BN>();
    constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        TI_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    int* status = ti_status_ptr();
    TI_REQUIRE(status != nullptr, "linear: no status word");
    dim3 grid((g.rows_a + BM - 1) / BM, (g.rows_b + BN - 1) / BN, g.splits);
    TI_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "linear: grid of %u x %u x %u is too large", grid.x, grid.y, grid.z);
    TI_CUDA(ti_launch_class<5>(gemm_tc_kernel<BN>, grid, dim3(THREADS), smem, stream, am, bm, g, status));
    TI_CHECK_LAUNCH("linear (tcgen05)");
    if (g.splits > 1 && !g.tickets) {
        const long long items = (long long)grid.x * grid.y * 4 * (BN / 16);
        const int warps = 4;
        TI_CUDA(ti_launch_class<5>(splitk_reduce_kernel<BN>, dim3((unsigned)((items + warps - 1) / warps)), dim3(warps * 32), 0, stream, g,
                          (int)grid.x, (int)grid.y));
        TI_CHECK_LAUNCH("linear (tcgen05, split reduction)");
    }
    return 0;
}
// How many tiles of a many-token product are shared out by contraction steps (TileWalk): with
// whole rounds of tiles, or less than one round, none; else the last round and the one before it,
// so that every unit's part is at least a tile long.
int shared_tiles_of(int tiles, int units) {
    if (units <= 0 || tiles < units || tiles % units == 0) return 0;
    return units + tiles % units;
}

template <int BN, bool PAIR>
int launch_walk(const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream) {
    constexpr int STAGES = walk_stages<BN, PAIR>();
    constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + (PAIR ? BN / 2 : BN) * BK * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        TI_CUDA(cudaFuncSetAttribute(gemm_tc_walk_kernel<BN, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    int* status = ti_status_ptr();
    TI_REQUIRE(status != nullptr, "linear: no status word");
    const int tile_rows = PAIR ? 2 * BM : BM;
    const int tiles = ((g.rows_a + tile_rows - 1) / tile_rows) * ((g.rows_b + BN - 1) / BN);
    const int all_units = PAIR ? sms / 2 : sms;
    const int units = g.shared_tiles > 0 || tiles > all_units ? all_units : tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(PAIR ? 2 * units : units);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (PAIR) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 2;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        n_attr++;
    }
    if (ti_pdl_enabled(5)) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    TI_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_walk_kernel<BN, PAIR>, am, bm, g, status));
    TI_CHECK_LAUNCH(PAIR ? "linear (tcgen05, two SMs per tile)" : "linear (tcgen05, tile walk)");
    return 0;
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
        if (g_pair_mode != 1 && pairs > 0 && tiles_a2 * tiles_b2 >= pairs && (useful >= 0.93 || g_pair_mode == 2)) {
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
    const int tile_rows = p.pair ? 2 * BM : BM;
    const int tiles = ((rows_a + tile_rows - 1) / tile_rows) * ((rows_b + b - 1) / b);
    int sp = 1;
    // measured with the weights as the row operand (16, 32, 64 tokens, the four products of a 4B-shaped
    // layer): 1.5 blocks per SM are 2-4 % faster in sum than 1.0, 2.0 are 10 % slower
    const int want = p.swap ? sms + sms / 2 : sms;
    if (tiles < want && !p.pair) {
        sp = (want + tiles / 2) / tiles;
        if (sp < 1) sp = 1;
        const int max_sp = nkb / 4 > 0 ? nkb / 4 : 1;       // at least four 64-wide blocks per split
        if (sp > max_sp) sp = max_sp;
        if (sp > 32) sp = 32;
        // drop splits that would get no work
        const int per = (nkb + sp - 1) / sp;
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
    if (int rc = operand_map(swap ? x : w, g.rows_b, K, swap ? ldx : ldw, p.pair ? bn / 2 : bn, &bm)) return rc;
    if (p.pair) return launch_walk<256, true>(am, bm, g, sms, stream);
    if (p.walk) {
        switch (bn) {
            case 128: return launch_walk<128, false>(am, bm, g, sms, stream);
            case 144: return launch_walk<144, false>(am, bm, g, sms, stream);
            case 160: return launch_walk<160, false>(am, bm, g, sms, stream);
            case 176: return launch_walk<176, false>(am, bm, g, sms, stream);
            case 192: return launch_walk<192, false>(am, bm, g, sms, stream);
            case 208: return launch_walk<208, false>(am, bm, g, sms, stream);
            case 224: return launch_walk<224, false>(am, bm, g, sms, stream);
            case 240: return launch_walk<240, false>(am, bm, g, sms, stream);
            default: return launch_walk<256, false>(am, bm, g, sms, stream);
        }
    }
    switch (bn) {
        case 16: return launch<16>(am, bm, g, stream);
        case 32: return launch<32>(am, bm, g, stream);
        case 64: return launch<64>(am, bm, g, stream);
        case 128: return launch<128>(am, bm, g, stream);
        case 144: return launch<144>(am, bm, g, stream);
        case 160: return launch<160>(am, bm, g, stream);
        case 176: return launch<176>(am, bm, g, stream);
        case 192: return launch<192>(am, bm, g, stream);
        case 208: return launch<208>(am, bm, g, stream);
        case 224: return launch<224>(am, bm, g, stream);
        case 240: return launch<240>(am, bm, g, stream);
        default: return launch<256>(am, bm, g, stream);
    }
}

// The many-token tcgen05 matrix product: the kernel and its launcher, instantiated by
// gemm_tcgen05_walk_{wide,mid,narrow}.cu (one SM per tile) and gemm_tcgen05_pair.cu (two).
#pragma once

#include "gemm_tcgen05.cuh"
#include "gemm_tile_walk.cuh"

namespace tigemm {
namespace {
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
//
// A pair also takes tiles wider than 256 weight rows (up to 512, BN a multiple of 32): two MMAs per
// step of the contraction, each BN / 2 columns wide, into one accumulator that fills the tensor
// memory; each block loads its quarter of the tile's weight rows for either MMA as a box of its
// own, so that the accumulator's columns follow the weight rows in order.  With one accumulator
// a tile's epilogue no longer runs under the next tile's MMAs: the form is for products whose
// tiles then fit the pairs in one round (2,048 x 2,560 outputs are 80 tiles of 256 x 256 for 74
// pairs but 72 of 256 x 288), where every pair walks the contraction from the same step at the
// same time and what one brings into L2 the others use: shared out by contraction steps instead,
// each pair starts at a step of its own and the L2 hit rate falls from 82 % to 62 %.
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

template <int BN, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_walk_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                    GemmArgs g, int* status) {
    ti_pdl_trigger();
    static_assert(BN <= 256 || (PAIR && BN % 32 == 0 && BN <= 512), "tiles wider than 256 weight rows: pairs only, a multiple of 32 up to 512");
    constexpr int STAGES = walk_stages<BN, PAIR>();
    constexpr int B_ROWS = PAIR ? BN / 2 : BN;                  // weight rows this block loads
    constexpr int N_MMA = BN > 256 ? 2 : 1;                     // MMAs per step of 16, each BN / N_MMA columns wide
    constexpr int MMA_N = BN / N_MMA;
    constexpr int B_BOX = B_ROWS / N_MMA;                       // weight rows per TMA box: this block's share of one MMA
    constexpr int N_ACC = BN > 256 ? 1 : 2;                     // accumulators in tensor memory
    constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;               // tokens of a tile
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = B_ROWS * BK * 2;
    constexpr uint32_t ACC_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : BN <= 256 ? 256 : 512;   // columns of one accumulator
    constexpr uint32_t TMEM_COLS = N_ACC * ACC_COLS;
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

    // The loading and the issuing thread are elected inside branches on a warp-uniform value: the
    // compiler then keeps their descriptors in uniform registers (see elect_one in tcgen05.cuh).
    const int warp_u = warp_uniform();
    if (warp_u == 0) {
        if (elect_one()) {
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
#pragma unroll
                        for (int h = 0; h < N_MMA; h++)     // MMA h reads weight rows h * MMA_N ...: this block brings its half of them
                            tma_load_2d_pair(sa + A_BYTES + h * (B_BOX * BK * 2), &b_map, kb * BK,
                                             b0 - rank * B_ROWS + h * MMA_N + rank * B_BOX, bar);
                    } else {
                        mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                        tma_load_2d(sa, &a_map, kb * BK, a0, &full[s]);
                        tma_load_2d(sa + A_BYTES, &b_map, kb * BK, b0, &full[s]);
                    }
                }
            }
        }
    } else if (warp_u == 1) {
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MMA_N >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
            int it = 0, n = 0;
            bool ok = true;
            TileWalk walk(g.shared_tiles, n_tiles, nkb, unit, units);
            Piece p;
            for (; ok && walk.next(p); n++) {
                const int buf = N_ACC == 2 ? n & 1 : 0, use = N_ACC == 2 ? n >> 1 : n;      // which accumulator, and its how-manieth use
                // the epilogue must have drained this accumulator (its use before this one)
                if (!mbar_wait(&acc_empty[buf], (uint32_t)((use & 1) ^ 1))) { ti_report(status, TI_STATUS_PIPE_WAIT); ok = false; break; }
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
                        if (PAIR) {
#pragma unroll
                            for (int h = 0; h < N_MMA; h++)     // a box of B_BOX rows of 128 bytes: whole groups of 8 rows, 1024 bytes each
                                tc_mma_bf16_pair(acc + h * MMA_N, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2 + ((h * B_BOX * BK * 2) >> 4)), idesc, accumulate);
                        }
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
            const int buf = N_ACC == 2 ? n & 1 : 0, use = N_ACC == 2 ? n >> 1 : n;
            int a0, b0;
            tile_origin(p.tile, tiles_a, tiles_b, TILE_ROWS, BN, a0, b0);
            const int i = a0 + rank * BM + q * 32 + lane;
            if (!mbar_wait(&acc_full[buf], (uint32_t)(use & 1))) { ti_report(status, TI_STATUS_MMA_WAIT); ok = false; }
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
            int other, other_place;
            TileWalk::other_piece(p.tile, nkb, unit, shared_steps, units, other, other_place);
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
                const float4* ws = reinterpret_cast<const float4*>(g.workspace + (((size_t)other * 2 + other_place) * blocks_per_unit + rank) * TILE_FLOATS) + t;
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
}  // namespace
}  // namespace tigemm

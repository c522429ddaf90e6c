// The tcgen05 matrix product with one block per tile: see gemm_tcgen05.cu for the whole picture.
#include "gemm_tcgen05.cuh"

namespace tigemm {
namespace {
// Narrow tiles (few tokens, the weights stream) keep five stages so that two blocks share an
// SM: a grid of about one block per SM then leaves room for the next kernel's blocks, which
// request their weights while this kernel is still running.  Wide tiles take the SM alone.
template <int BN> constexpr int stages_for() {
    constexpr int per = BM * BK * 2 + BN * BK * 2;
    constexpr int n = (200 * 1024) / per;
    return BN <= 32 ? 5 : BN == 64 ? 4 : (n > 8 ? 8 : n);
}
template <int BN> constexpr int blocks_per_sm() { return BN <= 64 ? 2 : 1; }

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
    // the loading and the issuing thread are elected inside branches on a warp-uniform value
    // (see elect_one in tcgen05.cuh)
    const int warp_u = warp_uniform();
    bool loader = false;
    if (warp_u == 0) loader = elect_one();
    if (loader) {
        for (int it = 0; it < n_pre; it++) {
            unsigned char* sa = smem + (size_t)it * (A_BYTES + B_BYTES);
            mbar_expect_tx(&full[it], A_BYTES + B_BYTES);
            if (weights_are_a) tma_load_2d(sa, &a_map, (kb0 + it) * BK, a0, &full[it]);
            else tma_load_2d(sa + A_BYTES, &b_map, (kb0 + it) * BK, b0, &full[it]);
        }
    }
    ti_pdl_sync();      // from here on memory written by earlier kernels may be read

    if (warp_u == 0) {
        // ---- TMA producer
        if (loader) {
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
    } else if (warp_u == 1) {
        // ---- MMA issuer
        if (elect_one()) {
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
}  // namespace

int launch_tile(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, cudaStream_t stream) {
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
}  // namespace tigemm

// What the translation units of the tcgen05 matrix product share: tile constants, the kernels'
// arguments, the epilogue's store, and the launchers each unit offers to the dispatcher in
// gemm_tcgen05.cu.  (The kernels are many template instances; split over files they compile
// side by side.)
#pragma once

#include "tcgen05.cuh"

namespace tigemm {
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

// One block per tile (few tokens with the weights as the row operand; few tiles with the
// contraction split): gemm_tcgen05_tile.cu.
int launch_tile(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, cudaStream_t stream);
// Every SM walking over tiles, one block per tile of 128 tokens (gemm_tcgen05_walk*.cu) or the two
// blocks of a cluster per tile of 256 (gemm_tcgen05_pair.cu); the kernel itself: gemm_tcgen05_walk.cuh.
int launch_walk_single(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream);
int launch_walk_pair(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream);
}  // namespace tigemm

// Warp-level tensor-core pieces shared by the attention kernels: ldmatrix, the
// m16n8k16 bfloat16 MMA with float32 accumulation, and the addressing of a tile that TMA
// stored as 64-column boxes under the 128-byte swizzle.
#pragma once

#include "common.cuh"

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of element (row, d) inside a tile of ROWS rows stored as boxes of
// [ROWS][128 bytes] (64 bfloat16 columns per box), 16-byte chunk c of row r at chunk c ^ (r % 8).
template <int ROWS>
__device__ __forceinline__ uint32_t swizzled_offset(int row, int d) {
    const int box = d >> 6, chunk = (d & 63) >> 3;
    return (uint32_t)(box * (ROWS * 128) + row * 128 + ((chunk ^ (row & 7)) << 4) + (d & 7) * 2);
}

// TMA and mbarrier helpers: tensor-map creation on the host, and the PTX wrappers the
// kernels use on the device.  Every wait is bounded: after `TI_SPIN_LIMIT` failed polls a
// wait gives up and returns false; the kernel then records a code in the library's status
// word (ti_read_status) and leaves without touching the data it was waiting for.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

#define TI_SPIN_LIMIT (1u << 24)

// status codes written by kernels (first failure wins)
#define TI_STATUS_OK 0
#define TI_STATUS_TMA_WAIT 1     // a wait for a TMA load ran out
#define TI_STATUS_MMA_WAIT 2     // a wait for tensor-core work ran out
#define TI_STATUS_PIPE_WAIT 3    // a wait for a pipeline slot ran out

// Device address of the library's status word (one per device), for kernels to report to.
int* ti_status_ptr();

__device__ __forceinline__ void ti_report(int* status, int code) { atomicCAS(status, 0, code); }

// ---------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------
// A 2-D bfloat16 tensor [rows, cols] with `row_stride_bytes` between rows, read in boxes of
// box_rows x box_cols (box_cols * 2 bytes must be 128 for the 128-byte swizzle).
int ti_make_tensor_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                               uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols);

// ---------------------------------------------------------------------------
// device: shared-memory addresses, mbarriers, TMA
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait; false when it gave up after `limit` polls.
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    return mbar_wait_limited(bar, parity, TI_SPIN_LIMIT);
}

// One box of a 2-D tensor map into shared memory; x is the inner (contiguous) coordinate and
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Host-side runtime pieces shared by the kernels: the status word that kernels report
// bounded-wait failures to, and tensor-map creation through the driver entry point
// (looked up at run time, so the library does not link against libcuda).
#include "tma.cuh"

#include <cudaTypedefs.h>

namespace {
__device__ int g_status_word = 0;

struct PerDevice { int* status = nullptr; };
PerDevice g_dev[64];

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int load_encode() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        ti_set_error("cuTensorMapEncodeTiled is not available from the driver: %s", cudaGetErrorString(e));
        return 2;
    }
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    return 0;
}
}  // namespace

static unsigned g_pdl_mask = ~0u;
int ti_pdl_enabled(int cls) { return (g_pdl_mask >> (cls & 31)) & 1u; }
// 0 switches programmatic dependent launch off (every kernel then starts after the one before
// it has ended), 1 switches it on again; the mask form sets it per class of kernels (bit = class).
extern "C" int ti_set_pdl(int on) { g_pdl_mask = on ? ~0u : 0u; return 0; }
extern "C" int ti_set_pdl_mask(unsigned mask) { g_pdl_mask = mask; return 0; }

int* ti_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!g_dev[dev].status) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        g_dev[dev].status = static_cast<int*>(p);
    }
    return g_dev[dev].status;
}

// Reads and clears the status word of the current device.  Synchronises the device.
extern "C" int ti_read_status(int* out) {
    int* p = ti_status_ptr();
    TI_REQUIRE(p != nullptr, "status word: no CUDA device");
    TI_CUDA(cudaDeviceSynchronize());
    TI_CUDA(cudaMemcpy(out, p, sizeof(int), cudaMemcpyDeviceToHost));
    if (*out != 0) TI_CUDA(cudaMemset(p, 0, sizeof(int)));
    return 0;
}

// ---------------------------------------------------------------------------
// A wait that runs out, on purpose and harmlessly: one block waits on an mbarrier in its own shared
// memory that nothing ever arrives on, with the given (small) number of polls instead of
// TI_SPIN_LIMIT, then does what every kernel of the library does when a wait gives up: it records
// the code in the status word and returns.  Nothing faults, traps or waits without a limit; the
// context stays usable.  For the test that checks how a run-out wait is reported; no product
// kernel's limit changes.
// ---------------------------------------------------------------------------
namespace {
__global__ void wait_runs_out_kernel(int* status, unsigned limit, int* gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const bool ok = mbar_wait_limited(&bar, 0, limit);
    if (!ok) ti_report(status, TI_STATUS_TMA_WAIT);
    if (threadIdx.x == 0 && gave_up) *gave_up = ok ? 0 : 1;
}
}  // namespace

extern "C" int ti_test_wait_runs_out(unsigned limit, int* gave_up, cudaStream_t stream) {
    TI_REQUIRE(limit >= 1 && limit <= (1u << 20), "wait test: the limit must be between 1 and 2^20 polls, got %u", limit);
    int* status = ti_status_ptr();
    TI_REQUIRE(status != nullptr, "wait test: no status word");
    wait_runs_out_kernel<<<1, 32, 0, stream>>>(status, limit, gave_up);
    TI_CHECK_LAUNCH("wait test");
    return 0;
}

int ti_make_tensor_map_2d_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                               uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols) {
    if (int rc = load_encode()) return rc;
    TI_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map: base address is not 16-byte aligned");
    TI_REQUIRE(row_stride_bytes % 16 == 0, "tensor map: row stride of %llu bytes is not a multiple of 16",
               (unsigned long long)row_stride_bytes);
    TI_REQUIRE(box_cols * 2 == 128 && box_rows >= 1 && box_rows <= 256, "tensor map: box of %u x %u is not supported",
               box_rows, box_cols);
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TI_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (rows %llu, cols %llu, stride %llu)", (int)r,
               (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)row_stride_bytes);
    return 0;
}

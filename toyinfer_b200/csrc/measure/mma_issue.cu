// A measurement, not a product kernel (built into a library of its own, libtoyinfer_measure.so,
// only when asked for): what one issuing thread per block gets out of the tensor
// cores.  Every block issues `batch` accumulating tcgen05 MMAs of 128 x N x 16 back to back, commits,
// waits (bounded) and repeats; the result is cycles per MMA as the issuing thread of block 0 sees
// them.  Operands are zeros in shared and tensor memory; nothing is read from or written to global
// memory but the result.  `python bench.py --kernel mma_issue` prints the table that decided how the
// kernels of this library choose their issuing thread (elect_one in tcgen05.cuh).
#include "../tcgen05.cuh"

#include <cstdarg>
#include <cstdio>

// this library's own error text (the kernels' library keeps its own)
static char g_error[512];
void ti_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}
extern "C" const char* ti_last_error() { return g_error; }

namespace {
// MODE 0: A and B in shared memory, both K-major (a first product Q K^T); 1: A in tensor memory, B
// K-major; 2: A in tensor memory, B MN-major (a second product P V); 3: A in shared memory, B MN-major.
template <int N, int MODE, bool ELECT>
__global__ void __launch_bounds__(128) mma_issue_kernel(int reps, int batch, long long* out) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    if (warp == 0) { __syncwarp(); tmem_alloc(&slot, 256); tmem_relinquish(); }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = slot;
    constexpr uint32_t DCOL = N == 256 ? 0 : 128;      // the accumulator; A, when in tensor memory, lies in columns 0 .. 63
    bool issuer = false;
    if (ELECT) { if (warp_uniform() == 0) issuer = elect_one(); }
    else issuer = threadIdx.x == 0;
    if (issuer) {
        constexpr uint32_t idesc = instr_desc_bf16(N, MODE >= 2);
        const uint64_t a_desc = smem_desc_sw128(smem_u32(smem));                      // 128 rows, two boxes of 64 columns
        const uint64_t bk_desc = smem_desc_sw128(smem_u32(smem + 32 * 1024));          // N rows, two boxes of 64 columns
        const uint64_t bm_desc = smem_desc_mn_sw128(smem_u32(smem + 32 * 1024), 64 * 128);
        long long total = 0, issue = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int r = 0; r < reps && ok; r++) {
            const long long t0 = clock64();
            for (int i = 0; i < batch; i++) {
                const int kk = i & 7;
                if (MODE == 0) tc_mma_bf16(tmem + DCOL, a_desc + (uint64_t)(((kk >> 2) * 128 * 128 + (kk & 3) * 32) >> 4),
                                           bk_desc + (uint64_t)(((kk >> 2) * N * 128 + (kk & 3) * 32) >> 4), idesc, i > 0);
                if (MODE == 1) tc_mma_bf16_ts(tmem + DCOL, tmem + kk * 8, bk_desc + (uint64_t)(((kk >> 2) * N * 128 + (kk & 3) * 32) >> 4), idesc, i > 0);
                if (MODE == 2) tc_mma_bf16_ts(tmem + DCOL, tmem + (kk & 3) * 8, bm_desc + (uint64_t)(((kk & 3) * 16 * 128) >> 4), idesc, i > 0);
                if (MODE == 3) tc_mma_bf16(tmem + DCOL, a_desc + (uint64_t)(((kk >> 2) * 128 * 128 + (kk & 3) * 32) >> 4),
                                           bm_desc + (uint64_t)(((kk & 3) * 16 * 128) >> 4), idesc, i > 0);
            }
            const long long t1 = clock64();
            tc_commit(&bar);
            ok = mbar_wait_limited(&bar, phase, 1u << 22);
            phase ^= 1;
            const long long t2 = clock64();
            if (r > 0) { total += t2 - t0; issue += t1 - t0; }      // the first round warms up
        }
        if (blockIdx.x == 0) { out[0] = ok ? total : -1; out[1] = (long long)(reps - 1) * batch; out[2] = issue; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 256); }
}

template <int N, int MODE, bool ELECT>
int run(int batch, int blocks, double* cycles, double* issue_cycles, cudaStream_t stream) {
    long long* out = nullptr;
    TI_CUDA(cudaMalloc(&out, 3 * sizeof(long long)));
    TI_CUDA(cudaMemsetAsync(out, 0, 3 * sizeof(long long), stream));
    const size_t smem = 100 * 1024;
    TI_CUDA(cudaFuncSetAttribute(mma_issue_kernel<N, MODE, ELECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mma_issue_kernel<N, MODE, ELECT><<<blocks, 128, smem, stream>>>(20, batch, out);
    TI_CHECK_LAUNCH("mma issue measurement");
    long long h[3] = {0, 0, 0};
    TI_CUDA(cudaMemcpyAsync(h, out, sizeof(h), cudaMemcpyDeviceToHost, stream));
    TI_CUDA(cudaStreamSynchronize(stream));
    TI_CUDA(cudaFree(out));
    TI_REQUIRE(h[0] > 0 && h[1] > 0, "mma issue measurement: a wait ran out");
    *cycles = (double)h[0] / (double)h[1];
    *issue_cycles = (double)h[2] / (double)h[1];
    return 0;
}
}  // namespace

// n: 64, 128 or 256 (256 only with mode 0); mode: see above; elect: how the issuing thread is chosen;
// blocks: how many blocks run it at once (one or two per SM make sense).
extern "C" int ti_bench_mma_issue(int n, int mode, int elect, int batch, int blocks, double* cycles, double* issue_cycles,
                                  cudaStream_t stream) {
    TI_REQUIRE(batch >= 1 && batch <= 4096 && blocks >= 1 && cycles && issue_cycles, "mma issue measurement: bad arguments");
#define TI_CASE(N_, M_) \
    if (n == N_ && mode == M_) return elect ? run<N_, M_, true>(batch, blocks, cycles, issue_cycles, stream) \
                                            : run<N_, M_, false>(batch, blocks, cycles, issue_cycles, stream);
    TI_CASE(64, 0) TI_CASE(64, 1) TI_CASE(128, 0) TI_CASE(128, 1) TI_CASE(128, 2) TI_CASE(128, 3) TI_CASE(256, 0)
#undef TI_CASE
    TI_FAIL("mma issue measurement: no case for N = %d, mode %d", n, mode);
}

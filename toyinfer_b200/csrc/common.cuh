// Shared device helpers and the error convention of the C entry points.
//
// Every entry point is `extern "C" int ti_<name>(..., cudaStream_t stream)`; it
// returns 0 on success and otherwise a non-zero code after storing a message that
// `ti_last_error()` returns.  Nothing here allocates device memory or synchronises.
// Element types are passed as codes: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TI_F32 0
#define TI_BF16 1

void ti_set_error(const char* fmt, ...);

#define TI_FAIL(...)                \
    do {                            \
        ti_set_error(__VA_ARGS__);  \
        return 1;                   \
    } while (0)

#define TI_REQUIRE(cond, ...)           \
    do {                                \
        if (!(cond)) {                  \
            ti_set_error(__VA_ARGS__);  \
            return 1;                   \
        }                               \
    } while (0)

#define TI_CHECK_LAUNCH(name)                                                          \
    do {                                                                               \
        cudaError_t e__ = cudaGetLastError();                                          \
        if (e__ != cudaSuccess) {                                                      \
            ti_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__));      \
            return 2;                                                                  \
        }                                                                              \
    } while (0)

#define TI_CUDA(call)                                                                  \
    do {                                                                               \
        cudaError_t e__ = (call);                                                      \
        if (e__ != cudaSuccess) {                                                      \
            ti_set_error("%s failed: %s", #call, cudaGetErrorString(e__));             \
            return 2;                                                                  \
        }                                                                              \
    } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `red` is shared memory for 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();  // protects `red` against a previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
    if (warp == 0) {
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Programmatic dependent launch: a kernel may be scheduled while the kernel before it in the
// stream still runs, so that its launch latency and set-up overlap that kernel's tail.  It
// must not touch global memory before `ti_pdl_sync()`, which waits until the earlier kernels
// have finished and their writes are visible.
// Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void ti_pdl_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// A pointer to what the kernel before this one wrote, to be used for loads after ti_pdl_sync().
// A load through a pointer that the compiler knows to be read-only for the whole kernel (a
// const __restrict__ parameter, __ldg) may be moved above any barrier, the wait included, and
// then reads what the earlier kernel has not written yet.  The pointer that comes out of this
// is the result of an asm statement that stays behind the wait, so loads through it do too.
template <typename T>
__device__ __forceinline__ T* ti_dependent(T* p) {
    asm volatile("" : "+l"(p) :: "memory");
    return p;
}

// Called first thing in every kernel: the next kernel in the stream may be scheduled as soon as
// all blocks of this one have started.  It still waits (ti_pdl_sync) for this kernel to finish
// before it reads anything this kernel or an earlier one wrote, so several kernels can sit on the
// SMs at once, each with its set-up done and its constant operands on the way.
__device__ __forceinline__ void ti_pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Whether kernels of a class start early (programmatic serialization) or only when everything
// before them in the stream has finished.  Classes: 0 everything not named below, 1 norms and
// other row-wise kernels, 2 rotate-and-store, 3 decode attention, 4 its combine, 5 tcgen05 product.
int ti_pdl_enabled(int cls);

// Launches `kernel` with the programmatic-serialization attribute (see ti_pdl_sync) when its
// class has it switched on.
template <int CLS, typename... KArgs, typename... Args>
static inline cudaError_t ti_launch_class(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                          Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ti_pdl_enabled(CLS) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
static inline cudaError_t ti_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    return ti_launch_class<0>(kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

// The same without the attribute: the kernel starts when everything before it in the stream
// has finished (its ti_pdl_sync() then returns at once).
template <typename... KArgs, typename... Args>
static inline cudaError_t ti_launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                          Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.numAttrs = 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename F>
static inline int ti_dispatch_dtype(int dtype, F&& f) {
    // f is called with a value of the element type
    if (dtype == TI_F32) return f(float());
    if (dtype == TI_BF16) return f(bf16());
    ti_set_error("unknown element type code %d", dtype);
    return 1;
}

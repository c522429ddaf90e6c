// Row-wise kernels: embedding gather, RMS norm (plain and fused with the residual
// sum), row gather with sum, and the SwiGLU activation.  All arithmetic is 32-bit;
// a value is rounded to the storage type exactly once, when it is written.
//
// Formulas follow the reference: gather src/prefill.cu:6-22; RMS norm
// src/decode.cu:99-125 and src/prefill.cu:74-94 (x * rsqrt(sum/n + eps) * w, no
// intermediate rounding); residual sum src/decode.cu:7-22; SwiGLU
// src/decode.cu:746-764 (up * gate / (1 + exp(-gate))).
#include "common.cuh"

#include <cstdarg>
#include <cstdio>

// ---------------------------------------------------------------------------
// error message storage (one per host thread)
// ---------------------------------------------------------------------------
static thread_local char g_error[1024] = "";

void ti_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* ti_last_error() { return g_error; }

// ---------------------------------------------------------------------------
// vector access: V elements of T at once when the row allows it
// ---------------------------------------------------------------------------
template <typename T, int V> struct Vec { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ void load_vec(const T* p, float* out) {
    if constexpr (V == 1) {
        out[0] = to_f32(p[0]);
    } else {
        struct alignas(sizeof(T) * V) Pack { T v[V]; };
        Pack pk = *reinterpret_cast<const Pack*>(p);
#pragma unroll
        for (int i = 0; i < V; i++) out[i] = to_f32(pk.v[i]);
    }
}

template <typename T, int V>
__device__ __forceinline__ void store_vec(T* p, const float* in) {
    if constexpr (V == 1) {
        p[0] = from_f32<T>(in[0]);
    } else {
        struct alignas(sizeof(T) * V) Pack { T v[V]; };
        Pack pk;
#pragma unroll
        for (int i = 0; i < V; i++) pk.v[i] = from_f32<T>(in[i]);
        *reinterpret_cast<Pack*>(p) = pk;
    }
}

template <typename T> constexpr int vec_width() { return 16 / sizeof(T); }

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------------------
// embedding gather: out[m, :] = table[ids[m], :] * scale; an id outside the table gives zeros.
// The reference gathers without a scale (src/prefill.cu:17-21); with scale == 1 the row is
// copied bit for bit, otherwise the product is formed in 32-bit and rounded once.
// ---------------------------------------------------------------------------
template <typename T, int V>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             T* __restrict__ out, int H, int vocab, float scale) {
    ti_pdl_trigger();
    ti_pdl_sync();
    ids = ti_dependent(ids);
    const int m = blockIdx.x;
    const int id = ids[m];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (size_t)(ok ? id : 0) * H;
    T* dst = out + (size_t)m * H;
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
        float x[V];
        load_vec<T, V>(src + i, x);
        if (!ok) {
#pragma unroll
            for (int j = 0; j < V; j++) x[j] = 0.f;
        }
        if (scale != 1.0f) {
#pragma unroll
            for (int j = 0; j < V; j++) x[j] *= scale;
        }
        store_vec<T, V>(dst + i, x);
    }
}

extern "C" int ti_embed(const void* table, const int* ids, void* out, int M, int H, int vocab,
                        float scale, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && H > 0 && vocab > 0, "embed: bad sizes M=%d H=%d vocab=%d", M, H, vocab);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        constexpr int V = vec_width<T>();
        const int threads = 128;
        if (H % V == 0 && aligned16(table) && aligned16(out))
            TI_CUDA(ti_launch_class<1>(embed_kernel<T, V>, dim3(M), dim3(threads), 0, stream, (const T*)table, ids, (T*)out, H, vocab, scale));
        else
            TI_CUDA(ti_launch_class<1>(embed_kernel<T, 1>, dim3(M), dim3(threads), 0, stream, (const T*)table, ids, (T*)out, H, vocab, scale));
        TI_CHECK_LAUNCH("embed");
        return 0;
    });
}

// ---------------------------------------------------------------------------
// float32 logits in place: x <- x * scale, then with cap > 0 the soft cap x <- cap * tanh(x / cap).
// (The reference has neither: its logits are the head product as it is, src/decode.cu:251-286.)
// ---------------------------------------------------------------------------
__global__ void logit_scale_cap_kernel(float* __restrict__ x, long long stride, int V, float scale, float cap) {
    ti_pdl_trigger();
    ti_pdl_sync();
    float* row = x + (size_t)blockIdx.y * stride;
    const float inv = cap > 0.f ? 1.0f / cap : 0.f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
        float v = row[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv);
        row[i] = v;
    }
}

extern "C" int ti_logit_scale_cap(float* logits, long long stride, int R, int V, float scale, float cap, cudaStream_t stream) {
    if (R == 0 || V == 0) return 0;
    TI_REQUIRE(R > 0 && V > 0 && stride >= V && R <= 65535, "logit_scale_cap: bad sizes R=%d V=%d stride=%lld", R, V, stride);
    TI_REQUIRE(cap >= 0.f, "logit_scale_cap: the cap must not be negative");
    const int threads = 256;
    const int bx = (V + threads - 1) / threads < 256 ? (V + threads - 1) / threads : 256;
    TI_CUDA(ti_launch_class<1>(logit_scale_cap_kernel, dim3(bx, R), dim3(threads), 0, stream, logits, stride, V, scale, cap));
    TI_CHECK_LAUNCH("logit_scale_cap");
    return 0;
}

// ---------------------------------------------------------------------------
// RMS norm of rows; with ADD, first h <- round(h + delta) in place and the norm is
// taken of the rounded sum (what the next reader of h sees).
// x rows may be strided (x_stride elements); out is dense.
// ---------------------------------------------------------------------------
template <typename T, typename W, int V, bool ADD>
__global__ void rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta,
                               const W* __restrict__ w, T* __restrict__ out, int H,
                               long long x_stride, float eps) {
    ti_pdl_trigger();
    __shared__ float red[33];
    ti_pdl_sync();
    x = ti_dependent(x); delta = ti_dependent(delta);
    const size_t row = blockIdx.x;
    T* xr = x + row * x_stride;
    const T* dr = ADD ? delta + row * (size_t)H : nullptr;
    T* orow = out + row * (size_t)H;
    float ss = 0.f;
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
        float a[V];
        load_vec<T, V>(xr + i, a);
        if constexpr (ADD) {
            float d[V];
            load_vec<T, V>(dr + i, d);
#pragma unroll
            for (int j = 0; j < V; j++) a[j] = to_f32(from_f32<T>(a[j] + d[j]));
            store_vec<T, V>(xr + i, a);
        }
#pragma unroll
        for (int j = 0; j < V; j++) ss = fmaf(a[j], a[j], ss);
    }
    ss = block_sum(ss, red);
    const float r = rsqrtf(fmaf(ss, 1.0f / (float)H, eps));
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
        float a[V], g[V];
        load_vec<T, V>(xr + i, a);  // the thread's own earlier store when ADD
        load_vec<W, V>(w + i, g);
#pragma unroll
        for (int j = 0; j < V; j++) a[j] = a[j] * r * g[j];
        store_vec<T, V>(orow + i, a);
    }
}

template <typename T, typename W, bool ADD>
static int launch_rmsnorm(void* x, const void* delta, const void* w, void* out, int M, int H,
                          long long x_stride, float eps, cudaStream_t stream) {
    constexpr int V = vec_width<T>();
    const bool vec = H % V == 0 && x_stride % V == 0 && aligned16(x) && aligned16(out) &&
                     aligned16(w) && (!ADD || aligned16(delta)) && sizeof(W) == sizeof(T);
    int threads = 256;
    if (H <= 256) threads = 64;
    else if (H <= 1024) threads = 128;
    if (vec)
        TI_CUDA(ti_launch_class<1>(rmsnorm_kernel<T, W, V, ADD>, dim3(M), dim3(threads), 0, stream, (T*)x, (const T*)delta,
                          (const W*)w, (T*)out, H, x_stride, eps));
    else
        TI_CUDA(ti_launch_class<1>(rmsnorm_kernel<T, W, 1, ADD>, dim3(M), dim3(threads), 0, stream, (T*)x, (const T*)delta,
                          (const W*)w, (T*)out, H, x_stride, eps));
    TI_CHECK_LAUNCH("rmsnorm");
    return 0;
}

// delta == nullptr: plain norm.  wdtype may be float32 while dtype is bfloat16.
extern "C" int ti_rmsnorm(void* x, const void* delta, const void* w, void* out, int M, int H,
                          long long x_stride, float eps, int dtype, int wdtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && H > 0, "rmsnorm: bad sizes M=%d H=%d", M, H);
    TI_REQUIRE(x_stride >= H, "rmsnorm: row stride %lld smaller than the row %d", x_stride, H);
    if (dtype == TI_F32) {
        TI_REQUIRE(wdtype == TI_F32, "rmsnorm: float32 rows need a float32 weight");
        return delta ? launch_rmsnorm<float, float, true>(x, delta, w, out, M, H, x_stride, eps, stream)
                     : launch_rmsnorm<float, float, false>(x, delta, w, out, M, H, x_stride, eps, stream);
    }
    TI_REQUIRE(dtype == TI_BF16, "rmsnorm: unknown element type code %d", dtype);
    if (wdtype == TI_BF16)
        return delta ? launch_rmsnorm<bf16, bf16, true>(x, delta, w, out, M, H, x_stride, eps, stream)
                     : launch_rmsnorm<bf16, bf16, false>(x, delta, w, out, M, H, x_stride, eps, stream);
    TI_REQUIRE(wdtype == TI_F32, "rmsnorm: unknown weight type code %d", wdtype);
    return delta ? launch_rmsnorm<bf16, float, true>(x, delta, w, out, M, H, x_stride, eps, stream)
                 : launch_rmsnorm<bf16, float, false>(x, delta, w, out, M, H, x_stride, eps, stream);
}

// ---------------------------------------------------------------------------
// out[r, :] = round(h[rows[r], :] + delta[rows[r], :])   (delta may be null)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gather_add_kernel(const T* __restrict__ h, const T* __restrict__ delta,
                                  const int* __restrict__ rows, T* __restrict__ out, int H, int M) {
    ti_pdl_trigger();
    ti_pdl_sync();
    h = ti_dependent(h); delta = ti_dependent(delta);
    const int r = blockIdx.x;
    const int src = rows[r];
    const bool ok = src >= 0 && src < M;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float a = 0.f;
        if (ok) {
            a = to_f32(h[(size_t)src * H + i]);
            if (delta) a = a + to_f32(delta[(size_t)src * H + i]);
        }
        out[(size_t)r * H + i] = from_f32<T>(a);
    }
}

extern "C" int ti_gather_add(const void* h, const void* delta, const int* rows, void* out, int R,
                             int H, int M, int dtype, cudaStream_t stream) {
    if (R == 0) return 0;
    TI_REQUIRE(R > 0 && H > 0 && M > 0, "gather_add: bad sizes R=%d H=%d M=%d", R, H, M);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        TI_CUDA(ti_launch_class<1>(gather_add_kernel<T>, dim3(R), dim3(256), 0, stream, (const T*)h, (const T*)delta, rows, (T*)out, H, M));
        TI_CHECK_LAUNCH("gather_add");
        return 0;
    });
}

// ---------------------------------------------------------------------------
// SwiGLU: gu[m, 0:I] = gate, gu[m, I:2I] = up; out[m, i] = up * gate / (1 + exp(-gate))
// ---------------------------------------------------------------------------
// gu[m, 2i] = gate_i, gu[m, 2i + 1] = up_i
template <typename T>
__global__ void swiglu_pairs_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, long long total) {
    ti_pdl_trigger();
    ti_pdl_sync();
    gu = ti_dependent(gu);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const float g = to_f32(gu[2 * idx]), u = to_f32(gu[2 * idx + 1]);
        out[idx] = from_f32<T>(u * (g / (1.0f + expf(-g))));
    }
}

template <typename T, int V>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, long long total_vecs) {
    ti_pdl_trigger();
    ti_pdl_sync();
    gu = ti_dependent(gu);
    const int per_row = I / V;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_vecs;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long m = idx / per_row;
        const int i = (int)(idx - m * per_row) * V;
        float g[V], u[V];
        load_vec<T, V>(gu + m * 2 * I + i, g);
        load_vec<T, V>(gu + m * 2 * I + I + i, u);
#pragma unroll
        for (int j = 0; j < V; j++) g[j] = u[j] * (g[j] / (1.0f + expf(-g[j])));
        store_vec<T, V>(out + m * I + i, g);
    }
}

extern "C" int ti_swiglu(const void* gu, void* out, int M, int I, int pairs, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(M > 0 && I > 0, "swiglu: bad sizes M=%d I=%d", M, I);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        constexpr int V = vec_width<T>();
        const int threads = 256;
        if (pairs) {
            const long long n = (long long)M * I;
            const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
            TI_CUDA(ti_launch_class<1>(swiglu_pairs_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (const T*)gu, (T*)out, I, n));
            TI_CHECK_LAUNCH("swiglu");
            return 0;
        }
        if (I % V == 0 && aligned16(gu) && aligned16(out)) {
            const long long n = (long long)M * (I / V);
            const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
            TI_CUDA(ti_launch_class<1>(swiglu_kernel<T, V>, dim3(blocks), dim3(threads), 0, stream, (const T*)gu, (T*)out, I, n));
        } else {
            const long long n = (long long)M * I;
            const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
            TI_CUDA(ti_launch_class<1>(swiglu_kernel<T, 1>, dim3(blocks), dim3(threads), 0, stream, (const T*)gu, (T*)out, I, n));
        }
        TI_CHECK_LAUNCH("swiglu");
        return 0;
    });
}

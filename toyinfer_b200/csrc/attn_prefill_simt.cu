// Causal grouped-query attention over the tokens of one step (sequences that start
// at position 0), CUDA cores, everything after the loads in 32-bit.  It is the
// attention of the 32-bit engine and the fallback of the bfloat16 engine for head
// sizes its tensor-core kernel does not take.
//
// For query i of a sequence: keys j <= i (and j > i - window when window > 0),
// s_ij = (q_i . k_j) * scale, online softmax with the running maximum subtracted
// before every exp, o_i = sum_j p_ij v_j / sum_j p_ij.  Query head h reads kv head
// h / (heads / kv_heads).  Reference: src/prefill.cu:224-379 (mask :316, grouping
// :265); unlike it, key tiles that the mask excludes entirely are skipped and the
// maximum is subtracted before exp (it rescales afterwards, src/prefill.cu:322,346).
//
// Grid (query tiles of 32, heads, sequences), 128 threads: thread t works on query
// row t/4; its 4 threads split the tile's 32 keys (scores) and the head's elements
// (output) between them.
#include "common.cuh"

namespace {
constexpr int BQ = 32, BKV = 32, THREADS = 128;

template <typename T, int MAXC>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    T* __restrict__ out, long long q_stride, long long k_stride, long long v_stride,
                    long long o_stride, const int* __restrict__ cu_new, int n_heads, int n_kv_heads,
                    int hd, float scale, int window) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    q = ti_dependent(q); k = ti_dependent(k); v = ti_dependent(v);
    const int ld = hd + 1;
    float* Qs = sm;
    float* Ks = Qs + BQ * ld;
    float* Vs = Ks + BKV * ld;
    float* Ps = Vs + BKV * ld;  // [BQ][BKV + 1]
    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BQ;
    const int tok0 = cu_new[b];
    const int n = cu_new[b + 1] - tok0;
    if (q0 >= n) return;
    const int kvh = h / (n_heads / n_kv_heads);
    const int t = threadIdx.x, r = t >> 2, c4 = t & 3;

    for (int idx = t; idx < BQ * hd; idx += THREADS) {
        const int rr = idx / hd, d = idx - rr * hd;
        Qs[rr * ld + d] = (q0 + rr < n) ? to_f32(q[(size_t)(tok0 + q0 + rr) * q_stride + (size_t)h * hd + d]) : 0.f;
    }
    float acc[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; c++) acc[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int qi = q0 + r;              // this thread's query position
    const int nc = hd >> 2;             // elements of the head per thread

    const int last_q = min(q0 + BQ, n) - 1;
    int kt_lo = 0;
    if (window > 0) kt_lo = max(0, q0 - window + 1) / BKV;
    const int kt_hi = last_q / BKV;
    for (int kt = kt_lo; kt <= kt_hi; kt++) {
        const int k0 = kt * BKV;
        __syncthreads();  // previous tile fully consumed (and Qs written, first time)
        for (int idx = t; idx < BKV * hd; idx += THREADS) {
            const int rr = idx / hd, d = idx - rr * hd;
            const bool ok = k0 + rr < n;
            const size_t tok = (size_t)(tok0 + k0 + rr);
            Ks[rr * ld + d] = ok ? to_f32(k[tok * k_stride + (size_t)kvh * hd + d]) : 0.f;
            Vs[rr * ld + d] = ok ? to_f32(v[tok * v_stride + (size_t)kvh * hd + d]) : 0.f;
        }
        __syncthreads();
        float s[8];
#pragma unroll
        for (int c = 0; c < 8; c++) s[c] = 0.f;
        const float* qrow = Qs + r * ld;
        for (int d = 0; d < hd; d++) {
            const float qv = qrow[d];
#pragma unroll
            for (int c = 0; c < 8; c++) s[c] = fmaf(qv, Ks[(c4 + 4 * c) * ld + d], s[c]);
        }
        float m_tile = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int kj = k0 + c4 + 4 * c;
            const bool ok = kj <= qi && kj < n && (window <= 0 || kj > qi - window);
            s[c] = ok ? s[c] * scale : -INFINITY;
            m_tile = fmaxf(m_tile, s[c]);
        }
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
        const float m_new = fmaxf(m_run, m_tile);
        float alpha = 1.f, l_tile = 0.f;
        if (m_new > -INFINITY) {
            alpha = expf(m_run - m_new);  // exp(-inf) = 0 on the first useful tile
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float p = expf(s[c] - m_new);
                Ps[r * (BKV + 1) + c4 + 4 * c] = p;
                l_tile += p;
            }
        } else {
#pragma unroll
            for (int c = 0; c < 8; c++) Ps[r * (BKV + 1) + c4 + 4 * c] = 0.f;
        }
        l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 1);
        l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 2);
        l_run = l_run * alpha + l_tile;
        m_run = m_new;
        __syncwarp();  // the four threads of a row are in one warp
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc) acc[c] *= alpha;
        const float* prow = Ps + r * (BKV + 1);
        for (int j = 0; j < BKV; j++) {
            const float p = prow[j];
            const float* vrow = Vs + j * ld + c4;
#pragma unroll
            for (int c = 0; c < MAXC; c++)
                if (c < nc) acc[c] = fmaf(p, vrow[4 * c], acc[c]);
        }
    }
    if (qi < n) {
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        T* orow = out + (size_t)(tok0 + qi) * o_stride + (size_t)h * hd;
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc) orow[c4 + 4 * c] = from_f32<T>(acc[c] * inv);
    }
}

template <typename T, int MAXC>
int launch(const void* q, const void* k, const void* v, void* out, long long qs, long long ks,
           long long vs, long long os, const int* cu_new, int n_seq, int max_new, int nh, int nkv,
           int hd, float scale, int window, cudaStream_t stream) {
    const size_t smem = ((size_t)(BQ + 2 * BKV) * (hd + 1) + (size_t)BQ * (BKV + 1)) * sizeof(float);
    static size_t configured = 0;
    if (smem > configured) {
        TI_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<T, MAXC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    dim3 grid((max_new + BQ - 1) / BQ, nh, n_seq);
    TI_CUDA(ti_launch(attn_prefill_kernel<T, MAXC>, grid, dim3(THREADS), smem, stream, (const T*)q, (const T*)k,
                      (const T*)v, (T*)out, qs, ks, vs, os, cu_new, nh, nkv, hd, scale, window));
    TI_CHECK_LAUNCH("attention_prefill");
    return 0;
}
}  // namespace

extern "C" int ti_attn_prefill_simt(const void* q, const void* k, const void* v, void* out,
                                    long long q_stride, long long k_stride, long long v_stride,
                                    long long o_stride, const int* cu_new, int n_seq, int max_new,
                                    int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                    int dtype, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(n_seq > 0 && max_new > 0 && n_heads > 0 && n_kv_heads > 0, "attention_prefill: bad sizes");
    TI_REQUIRE(n_heads % n_kv_heads == 0, "attention_prefill: %d heads over %d kv heads", n_heads, n_kv_heads);
    TI_REQUIRE(head_dim % 4 == 0 && head_dim >= 4 && head_dim <= 256,
               "attention_prefill: head size %d not supported (multiples of 4 up to 256)", head_dim);
    TI_REQUIRE(n_seq <= 65535 && n_heads <= 65535, "attention_prefill: too many sequences or heads for one launch");
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        if (head_dim <= 64)
            return launch<T, 16>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new,
                                 n_heads, n_kv_heads, head_dim, scale, window, stream);
        if (head_dim <= 128)
            return launch<T, 32>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new,
                                 n_heads, n_kv_heads, head_dim, scale, window, stream);
        return launch<T, 64>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new,
                             n_heads, n_kv_heads, head_dim, scale, window, stream);
    });
}

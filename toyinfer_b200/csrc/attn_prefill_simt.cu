// Causal grouped-query attention of the tokens of one step, CUDA cores, everything
// after the loads in 32-bit.  It is the attention of the 32-bit engine and the
// fallback of the bfloat16 engine for head sizes its tensor-core kernels do not take.
//
// For the query at position i of a sequence: keys j <= i (and j > i - window when
// window > 0), s_ij = (q_i . k_j) * scale, online softmax with the running maximum
// subtracted before every exp, o_i = sum_j p_ij v_j / sum_j p_ij.  Query head h reads
// kv head h / (heads / kv_heads).  Reference: src/prefill.cu:224-379 (mask :316,
// grouping :265); unlike it, key tiles that the mask excludes entirely are skipped and
// the maximum is subtracted before exp (it rescales afterwards, src/prefill.cu:322,346).
//
// Two forms.  In the first every sequence starts at position 0 and all keys are the
// step's own.  In the second (PAGED) a sequence's new tokens follow `seq_start[b]`
// positions that earlier steps left in the paged cache: keys at positions below the
// start are read from the sequence's pages (position p at row p, or p mod ring_rows in a
// windowed group), keys from the start on from the step's own k and v; the cache is not
// asked for anything this step writes.  The reference cannot continue a sequence by more
// than one token (src/prefill.cu:185-208 rotates with position = token index,
// src/transformer.cpp:393-398 always writes cache rows [0, T)).
//
// Grid (query tiles of 32, heads, sequences), 128 threads: thread t works on query
// row t/4; its 4 threads split the tile's 32 keys (scores) and the head's elements
// (output) between them.
#include "common.cuh"

namespace {
constexpr int BQ = 32, BKV = 32, THREADS = 128;

// Where earlier positions of the step's sequences are kept (PAGED form only).
struct PagedKV {
    const void* k_pages; const void* v_pages;      // [pages, kv_heads, page_size, head_dim]
    const int* page_table; int table_width; int page_size; int ring_rows; int n_pages;
    const int* seq_start; const int* seq_slot;
};

template <typename T, int MAXC, bool PAGED>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    T* __restrict__ out, long long q_stride, long long k_stride, long long v_stride,
                    long long o_stride, const int* __restrict__ cu_new, int n_heads, int n_kv_heads,
                    int hd, float scale, int window, PagedKV kv) {
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
    // positions are counted from the sequence's first token; the step's tokens begin at `start`
    const int start = PAGED ? kv.seq_start[b] : 0;
    const int slot = PAGED ? kv.seq_slot[b] : 0;
    const int end = start + n;

    for (int idx = t; idx < BQ * hd; idx += THREADS) {
        const int rr = idx / hd, d = idx - rr * hd;
        Qs[rr * ld + d] = (q0 + rr < n) ? to_f32(q[(size_t)(tok0 + q0 + rr) * q_stride + (size_t)h * hd + d]) : 0.f;
    }
    float acc[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; c++) acc[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const int qi = start + q0 + r;      // this thread's query position
    const int nc = hd >> 2;             // elements of the head per thread

    const int last_q = start + min(q0 + BQ, n) - 1;
    const int lo_blk = window > 0 ? max(0, start + q0 - window + 1) : 0;     // oldest key any query of the tile reads
    const int kt_lo = lo_blk / BKV;
    const int kt_hi = last_q / BKV;
    for (int kt = kt_lo; kt <= kt_hi; kt++) {
        const int k0 = kt * BKV;
        __syncthreads();  // previous tile fully consumed (and Qs written, first time)
        for (int idx = t; idx < BKV * hd; idx += THREADS) {
            const int rr = idx / hd, d = idx - rr * hd;
            const int p = k0 + rr;
            float kx = 0.f, vx = 0.f;
            if (p >= start) {
                if (p < end) {
                    const size_t tok = (size_t)(tok0 + p - start);
                    kx = to_f32(k[tok * k_stride + (size_t)kvh * hd + d]);
                    vx = to_f32(v[tok * v_stride + (size_t)kvh * hd + d]);
                }
            } else if (PAGED && p >= lo_blk) {
                // a line outside [lo_blk, start) may hold anything and is never read
                const int row = kv.ring_rows > 0 ? p % kv.ring_rows : p;
                const int pidx = row / kv.page_size;
                const int page = pidx < kv.table_width ? kv.page_table[(size_t)slot * kv.table_width + pidx] : -1;
                if (page >= 0 && page < kv.n_pages) {
                    const size_t off = (((size_t)page * n_kv_heads + kvh) * kv.page_size + row % kv.page_size) * hd + d;
                    kx = to_f32(((const T*)kv.k_pages)[off]);
                    vx = to_f32(((const T*)kv.v_pages)[off]);
                }
            }
            Ks[rr * ld + d] = kx;
            Vs[rr * ld + d] = vx;
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
            const bool ok = kj <= qi && kj < end && (window <= 0 || kj > qi - window);
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
    if (qi < end) {
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        T* orow = out + (size_t)(tok0 + qi - start) * o_stride + (size_t)h * hd;
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nc) orow[c4 + 4 * c] = from_f32<T>(acc[c] * inv);
    }
}

template <typename T, int MAXC, bool PAGED>
int launch(const void* q, const void* k, const void* v, void* out, long long qs, long long ks,
           long long vs, long long os, const int* cu_new, int n_seq, int max_new, int nh, int nkv,
           int hd, float scale, int window, const PagedKV& c, cudaStream_t stream) {
    const size_t smem = ((size_t)(BQ + 2 * BKV) * (hd + 1) + (size_t)BQ * (BKV + 1)) * sizeof(float);
    static size_t configured = 0;
    if (smem > configured) {
        TI_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<T, MAXC, PAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    dim3 grid((max_new + BQ - 1) / BQ, nh, n_seq);
    TI_CUDA(ti_launch(attn_prefill_kernel<T, MAXC, PAGED>, grid, dim3(THREADS), smem, stream, (const T*)q, (const T*)k,
                      (const T*)v, (T*)out, qs, ks, vs, os, cu_new, nh, nkv, hd, scale, window, c));
    TI_CHECK_LAUNCH(PAGED ? "attention_chunk" : "attention_prefill");
    return 0;
}

template <bool PAGED>
int run(const void* q, const void* k, const void* v, void* out, long long q_stride, long long k_stride,
        long long v_stride, long long o_stride, const int* cu_new, int n_seq, int max_new, int n_heads,
        int n_kv_heads, int head_dim, float scale, int window, const PagedKV& c, int dtype, cudaStream_t stream) {
    const char* what = PAGED ? "attention_chunk" : "attention_prefill";
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(n_seq > 0 && max_new > 0 && n_heads > 0 && n_kv_heads > 0, "%s: bad sizes", what);
    TI_REQUIRE(n_heads % n_kv_heads == 0, "%s: %d heads over %d kv heads", what, n_heads, n_kv_heads);
    TI_REQUIRE(head_dim % 4 == 0 && head_dim >= 4 && head_dim <= 256,
               "%s: head size %d not supported (multiples of 4 up to 256)", what, head_dim);
    TI_REQUIRE(n_seq <= 65535 && n_heads <= 65535, "%s: too many sequences or heads for one launch", what);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        if (head_dim <= 64)
            return launch<T, 16, PAGED>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new,
                                        n_heads, n_kv_heads, head_dim, scale, window, c, stream);
        if (head_dim <= 128)
            return launch<T, 32, PAGED>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new,
                                        n_heads, n_kv_heads, head_dim, scale, window, c, stream);
        return launch<T, 64, PAGED>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new,
                                    n_heads, n_kv_heads, head_dim, scale, window, c, stream);
    });
}
}  // namespace

extern "C" int ti_attn_prefill_simt(const void* q, const void* k, const void* v, void* out,
                                    long long q_stride, long long k_stride, long long v_stride,
                                    long long o_stride, const int* cu_new, int n_seq, int max_new,
                                    int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                    int dtype, cudaStream_t stream) {
    return run<false>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new, n_heads,
                      n_kv_heads, head_dim, scale, window, PagedKV{}, dtype, stream);
}

// The step's tokens after `seq_start[b]` positions that the cache holds: q[M, heads, d], k and
// v[M, kv_heads, d] are the step's own (normed and rotated; whether they are in the cache yet does
// not matter, the cache is read below the start only).
extern "C" int ti_attn_chunk_simt(const void* q, const void* k, const void* v, void* out,
                                  long long q_stride, long long k_stride, long long v_stride,
                                  long long o_stride, const int* cu_new, const int* seq_start, const int* seq_slot,
                                  int n_seq, int max_new, int n_heads, int n_kv_heads, int head_dim, float scale,
                                  int window, const void* k_pages, const void* v_pages, const int* page_table,
                                  int table_width, int page_size, int ring_rows, int n_pages, int dtype,
                                  cudaStream_t stream) {
    TI_REQUIRE(k_pages && v_pages && page_table && seq_start && seq_slot && page_size > 0 && table_width > 0 && n_pages > 0,
               "attention_chunk: incomplete cache description");
    TI_REQUIRE(ring_rows % page_size == 0, "attention_chunk: ring of %d rows is not whole pages", ring_rows);
    TI_REQUIRE(ring_rows == 0 || (window > 0 && ring_rows >= window),
               "attention_chunk: a ring of %d rows needs a window of at most as many positions (got %d)", ring_rows, window);
    PagedKV c{k_pages, v_pages, page_table, table_width, page_size, ring_rows, n_pages, seq_start, seq_slot};
    return run<true>(q, k, v, out, q_stride, k_stride, v_stride, o_stride, cu_new, n_seq, max_new, n_heads,
                     n_kv_heads, head_dim, scale, window, c, dtype, stream);
}

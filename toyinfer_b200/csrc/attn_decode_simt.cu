// Grouped-query attention of one new token per sequence over the paged cache,
// split along the keys, CUDA cores, 32-bit arithmetic.
//
// For sequence b with length L (the new token included, already stored) and query
// head h: keys at positions max(0, L - window) .. L-1 (all of them when window == 0),
// s_j = (q . k_j) * scale, softmax with the maximum subtracted, o = sum p_j v_j.
// Reference: src/decode.cu:401-432 (scores), :471-532 (softmax), :598-628 (values);
// it materialises all scores and clears max_seq_len-sized buffers every layer
// (src/decode.cu:703-744), here nothing is proportional to the capacity.
//
// Grid (sequences, kv heads, splits), 128 threads.  A block takes the query heads
// that share its kv head, so every key and value is read once for all of them.  The
// tiles of 64 positions in range are dealt to the splits in contiguous runs; a tile
// is one page of the cache.  Each split writes an unnormalised partial result with
// its maximum and sum; `attn_decode_combine_kernel` merges them.  With one split the
// result is written directly.
#include "attn_decode.cuh"

namespace {
using tiattn::DecodeArgs;
using tiattn::attn_decode_combine_kernel;
constexpr int TILE = 64, THREADS = 128, MAXACC = 32;

template <typename T>
__global__ void __launch_bounds__(THREADS) attn_decode_kernel(DecodeArgs a) {
    ti_pdl_trigger();
    extern __shared__ float sm[];
    ti_pdl_sync();
    const int hd = a.hd, ld = hd + 1;
    const int g = a.n_heads / a.n_kv_heads;
    float* Qs = sm;                    // [g][hd]
    float* Ks = Qs + g * hd;           // [TILE][ld]
    float* Vs = Ks + TILE * ld;        // [TILE][hd]
    float* Ss = Vs + TILE * hd;        // [g][TILE]
    float* Mh = Ss + g * TILE;         // [g] running max
    float* Lh = Mh + g;                // [g] running sum
    float* Ah = Lh + g;                // [g] rescale of this tile
    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int L = a.seq_len[b];
    const int slot = a.seq_slot[b];
    const int lo = a.window > 0 ? max(0, L - a.window) : 0;
    const int tile_lo = lo / TILE, tile_hi = (L - 1) / TILE;       // inclusive
    const int n_tiles = L > 0 ? tile_hi - tile_lo + 1 : 0;
    const int per = (n_tiles + a.n_splits - 1) / a.n_splits;
    const int my_lo = tile_lo + split * per;
    const int my_hi = min(my_lo + per, tile_lo + n_tiles);           // exclusive
    const int h0 = kvh * g;

    for (int idx = t; idx < g * hd; idx += THREADS)
        Qs[idx] = to_f32(((const T*)a.q)[(size_t)b * a.q_stride + (size_t)h0 * hd + idx]);
    if (t < g) { Mh[t] = -INFINITY; Lh[t] = 0.f; }
    float acc[MAXACC];
#pragma unroll
    for (int c = 0; c < MAXACC; c++) acc[c] = 0.f;
    const int n_out = g * hd;

    for (int tile = my_lo; tile < my_hi; tile++) {
        const int p0 = tile * TILE;
        const int row0 = a.ring_rows > 0 ? p0 % a.ring_rows : p0;
        const int pidx = row0 / a.page_size;
        int page = pidx < a.table_width ? a.page_table[(size_t)slot * a.table_width + pidx] : 0;
        if (page < 0 || page >= a.n_pages) page = 0;
        const T* kp = (const T*)a.k_pages + ((size_t)page * a.n_kv_heads + kvh) * a.page_size * hd;
        const T* vp = (const T*)a.v_pages + ((size_t)page * a.n_kv_heads + kvh) * a.page_size * hd;
        __syncthreads();  // previous tile consumed; Qs/Mh/Lh written (first time)
        for (int idx = t; idx < TILE * hd; idx += THREADS) {
            const int j = idx / hd, d = idx - j * hd;
            const bool live = p0 + j >= lo && p0 + j < L;   // a line outside the range may hold anything
            Ks[j * ld + d] = live ? to_f32(kp[idx]) : 0.f;
            Vs[idx] = live ? to_f32(vp[idx]) : 0.f;
        }
        __syncthreads();
        for (int idx = t; idx < g * TILE; idx += THREADS) {
            const int gi = idx / TILE, j = idx - gi * TILE;
            const int p = p0 + j;
            float s = -INFINITY;
            if (p >= lo && p < L) {
                s = 0.f;
                const float* qv = Qs + gi * hd;
                const float* kv = Ks + j * ld;
                for (int d = 0; d < hd; d++) s = fmaf(qv[d], kv[d], s);
                s *= a.scale;
            }
            Ss[idx] = s;
        }
        __syncthreads();
        for (int gi = warp; gi < g; gi += THREADS / 32) {
            const float s0 = Ss[gi * TILE + lane], s1 = Ss[gi * TILE + 32 + lane];
            const float m_old = Mh[gi];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
            float p0v = 0.f, p1v = 0.f, alpha = 1.f;
            if (m_new > -INFINITY) {
                p0v = expf(s0 - m_new);
                p1v = expf(s1 - m_new);
                alpha = expf(m_old - m_new);
            }
            Ss[gi * TILE + lane] = p0v;
            Ss[gi * TILE + 32 + lane] = p1v;
            const float l_tile = warp_sum(p0v + p1v);
            if (lane == 0) { Mh[gi] = m_new; Lh[gi] = Lh[gi] * alpha + l_tile; Ah[gi] = alpha; }
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < MAXACC; c++) {
            const int idx = t + c * THREADS;
            if (idx < n_out) {
                const int gi = idx / hd, d = idx - gi * hd;
                float o = acc[c] * Ah[gi];
                const float* pr = Ss + gi * TILE;
                for (int j = 0; j < TILE; j++) o = fmaf(pr[j], Vs[j * hd + d], o);
                acc[c] = o;
            }
        }
    }
    __syncthreads();
    if (a.n_splits == 1) {
#pragma unroll
        for (int c = 0; c < MAXACC; c++) {
            const int idx = t + c * THREADS;
            if (idx < n_out) {
                const int gi = idx / hd, d = idx - gi * hd;
                const float l = Lh[gi];
                ((T*)a.out)[(size_t)b * a.o_stride + (size_t)(h0 + gi) * hd + d] = from_f32<T>(l > 0.f ? acc[c] / l : 0.f);
            }
        }
        return;
    }
#pragma unroll
    for (int c = 0; c < MAXACC; c++) {
        const int idx = t + c * THREADS;
        if (idx < n_out) {
            const int gi = idx / hd, d = idx - gi * hd;
            a.part_o[(((size_t)b * a.n_heads + h0 + gi) * a.n_splits + split) * hd + d] = acc[c];
        }
    }
    if (t < g) {
        float* ml = a.part_ml + (((size_t)b * a.n_heads + h0 + t) * a.n_splits + split) * 2;
        ml[0] = Mh[t];
        ml[1] = Lh[t];
    }
}

template <typename T>
int launch(const DecodeArgs& a, int n_seq, cudaStream_t stream) {
    const int g = a.n_heads / a.n_kv_heads, hd = a.hd;
    const size_t smem = ((size_t)g * hd + (size_t)TILE * (hd + 1) + (size_t)TILE * hd + (size_t)g * TILE + 3 * g) * sizeof(float);
    TI_REQUIRE(smem <= 227 * 1024, "attention_decode: %d query heads per kv head of size %d need %zu bytes of shared memory",
               g, hd, smem);
    static size_t configured = 0;
    if (smem > configured) {
        TI_CUDA(cudaFuncSetAttribute(attn_decode_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    dim3 grid(n_seq, a.n_kv_heads, a.n_splits);
    TI_CUDA(ti_launch(attn_decode_kernel<T>, grid, dim3(THREADS), smem, stream, a));
    TI_CHECK_LAUNCH("attention_decode");
    if (a.n_splits > 1) {
        dim3 cgrid(n_seq, a.n_heads);
        TI_CUDA(ti_launch(attn_decode_combine_kernel<T>, cgrid, dim3(hd < 128 ? 64 : 128), 0, stream, (const float*)a.part_o, (const float*)a.part_ml, (T*)a.out, a.o_stride, a.n_heads, hd, a.n_splits));
        TI_CHECK_LAUNCH("attention_decode (combine)");
    }
    return 0;
}
}  // namespace

// part_o needs n_seq*n_heads*n_splits*head_dim floats and part_ml n_seq*n_heads*n_splits*2
// (both unused when n_splits == 1).
extern "C" int ti_attn_decode_simt(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                   const int* page_table, int table_width, int page_size, int ring_rows,
                                   int n_pages, const int* seq_slot, const int* seq_len, int n_seq,
                                   int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                   int n_splits, void* out, long long o_stride, float* part_o,
                                   float* part_ml, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention_decode: bad head counts");
    TI_REQUIRE(head_dim > 0 && head_dim <= 512, "attention_decode: head size %d not supported", head_dim);
    TI_REQUIRE(page_size == TILE, "attention_decode: pages of %d positions, this kernel works on %d", page_size, TILE);
    TI_REQUIRE(ring_rows % page_size == 0, "attention_decode: ring of %d rows is not whole pages", ring_rows);
    TI_REQUIRE(window == 0 || ring_rows == 0 || ring_rows >= window, "attention_decode: ring of %d rows is smaller than the window %d", ring_rows, window);
    TI_REQUIRE((n_heads / n_kv_heads) * head_dim <= MAXACC * THREADS,
               "attention_decode: %d query heads per kv head of size %d exceed this kernel's %d outputs per block",
               n_heads / n_kv_heads, head_dim, MAXACC * THREADS);
    TI_REQUIRE(n_splits >= 1 && n_splits <= 65535 && n_kv_heads <= 65535, "attention_decode: bad split count %d", n_splits);
    TI_REQUIRE(n_splits == 1 || (part_o && part_ml), "attention_decode: split results need scratch memory");
    DecodeArgs a;
    a.q = q; a.q_stride = q_stride; a.k_pages = k_pages; a.v_pages = v_pages; a.page_table = page_table;
    a.table_width = table_width; a.page_size = page_size; a.ring_rows = ring_rows; a.n_pages = n_pages;
    a.seq_slot = seq_slot; a.seq_len = seq_len; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim;
    a.window = window; a.n_splits = n_splits; a.scale = scale; a.out = out; a.o_stride = o_stride;
    a.part_o = part_o; a.part_ml = part_ml;
    return ti_dispatch_dtype(dtype, [&](auto t) -> int { return launch<decltype(t)>(a, n_seq, stream); });
}

// ---------------------------------------------------------------------------
// The same kernels with their scratch inside the library (see attn_decode_noalloc.h).
// ---------------------------------------------------------------------------
#include "attn_decode_noalloc.h"

// Partial outputs first, then the (maximum, sum) pairs.  In host code this name is only a
// handle for the runtime; the address kernels can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[TI_NOALLOC_SCRATCH_FLOATS];

namespace {
float* g_noalloc_ptr[64] = {nullptr};   // per device, looked up at the first call on it

int noalloc_scratch(float** out) {
    int dev = 0;
    TI_CUDA(cudaGetDevice(&dev));
    TI_REQUIRE(dev >= 0 && dev < 64, "attention_decode (no allocation): device %d out of range", dev);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        TI_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
        TI_REQUIRE(p != nullptr, "attention_decode (no allocation): the scratch array has no device address");
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}
}  // namespace

extern "C" int ti_attn_decode_noalloc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                      const int* page_table, int table_width, int page_size, int ring_rows,
                                      int n_pages, const int* seq_slot, const int* seq_len, int n_seq,
                                      int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                      int n_splits, void* out, long long o_stride, int dtype, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(n_seq > 0 && n_heads > 0 && head_dim > 0 && n_splits >= 1, "attention_decode (no allocation): bad sizes");
    if (n_splits == 1)      // one split writes its result directly: no scratch is touched, and none is looked up
        return ti_attn_decode_simt(q, q_stride, k_pages, v_pages, page_table, table_width, page_size, ring_rows, n_pages,
                                   seq_slot, seq_len, n_seq, n_heads, n_kv_heads, head_dim, scale, window, 1, out,
                                   o_stride, nullptr, nullptr, dtype, stream);
    const long long need = (long long)n_seq * n_heads * n_splits * (head_dim + 2);
    TI_REQUIRE(need <= (long long)TI_NOALLOC_SCRATCH_FLOATS,
               "attention_decode (no allocation): %d sequences x %d heads x %d splits x head size %d need %lld floats of "
               "scratch, the library holds %d; use fewer splits or sequences per call, or the entry point that takes scratch",
               n_seq, n_heads, n_splits, head_dim, need, TI_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (int rc = noalloc_scratch(&scratch)) return rc;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)n_seq * n_heads * n_splits * head_dim;
    return ti_attn_decode_simt(q, q_stride, k_pages, v_pages, page_table, table_width, page_size, ring_rows, n_pages,
                               seq_slot, seq_len, n_seq, n_heads, n_kv_heads, head_dim, scale, window, n_splits, out,
                               o_stride, part_o, part_ml, dtype, stream);
}

// Per-head RMS norm of q and k, rotary encoding, and the store of k and v into the
// paged cache, in one pass over the projection's output.  Each stage is optional:
// a null norm weight skips the norm, null tables skip the rotation, null pages skip
// the store, a null q/k/v pointer skips that tensor.
//
// Reference formulas: per-head norm src/decode.cu:144-187 (one [head_dim] weight for
// all heads, rounded to the storage type before the rotation, as its in-place kernel
// does); rotation src/decode.cu:301-324 (pairs i, i + head_dim/2); cache row write
// src/decode.cu:374-386.  The reference runs these as five launches plus two copies
// per layer (src/transformer.cpp:380-398, :535-552).
//
// One warp handles one (token, head).  The cache position of a token:
//   row  = pos                    (ring_rows == 0)
//   row  = pos mod ring_rows      (windowed group; tokens older than the ring are not stored)
//   page = page_table[slot][row / page_size], line row % page_size
#include "rope_math.cuh"

#include <type_traits>

struct RopeStoreArgs {
    void* q; void* k; void* v;
    long long q_stride, k_stride, v_stride;   // elements between consecutive tokens
    int n_heads, n_kv_heads, head_dim;
    const void* q_w; const void* k_w; int w_is_f32; float eps;
    const float* cos_t; const float* sin_t; int max_pos;
    const int* tok_pos; const int* tok_seq; const int* seq_slot; const int* seq_len;
    void* k_pages; void* v_pages; const int* page_table; int table_width; int page_size;
    int ring_rows; int n_pages;
    int M;
};

template <typename T>
__global__ void rope_store_kernel(RopeStoreArgs a) {
    ti_pdl_trigger();
    ti_pdl_sync();
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int heads_q = a.q ? a.n_heads : 0;
    const int heads_k = a.k ? a.n_kv_heads : 0;
    const int heads_v = a.v ? a.n_kv_heads : 0;
    const int per_tok = heads_q + heads_k + heads_v;
    const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (item >= (long long)a.M * per_tok) return;
    const int m = (int)(item / per_tok);
    int h = (int)(item - (long long)m * per_tok);
    int kind;  // 0 q, 1 k, 2 v
    if (h < heads_q) kind = 0;
    else if (h < heads_q + heads_k) { kind = 1; h -= heads_q; }
    else { kind = 2; h -= heads_q + heads_k; }

    const int hd = a.head_dim, half = hd >> 1;
    T* x = kind == 0 ? (T*)a.q + (size_t)m * a.q_stride + (size_t)h * hd
         : kind == 1 ? (T*)a.k + (size_t)m * a.k_stride + (size_t)h * hd
                     : (T*)a.v + (size_t)m * a.v_stride + (size_t)h * hd;
    int pos = a.tok_pos[m];

    // where the cache keeps this token, if it does
    T* dst = nullptr;
    if (kind != 0 && a.k_pages) {
        const int seq = a.tok_seq[m];
        const int slot = a.seq_slot[seq];
        int row = pos;
        bool keep = pos >= 0;
        if (a.ring_rows > 0) {
            keep = keep && pos >= a.seq_len[seq] - a.ring_rows;
            row = pos % a.ring_rows;
        }
        const int pidx = row / a.page_size;
        if (keep && pidx < a.table_width) {
            const int page = a.page_table[(size_t)slot * a.table_width + pidx];
            if (page >= 0 && page < a.n_pages) {
                T* base = (T*)(kind == 1 ? a.k_pages : a.v_pages);
                dst = base + (((size_t)page * a.n_kv_heads + h) * a.page_size + (row % a.page_size)) * hd;
            }
        }
    }

    if (kind == 2) {  // values: copy only
        if (dst)
            for (int i = lane; i < hd; i += 32) dst[i] = x[i];
        return;
    }

    const void* wv = kind == 0 ? a.q_w : a.k_w;
    float r = 1.f;
    if (wv) {
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) {
            const float t = to_f32(x[i]);
            ss = fmaf(t, t, ss);
        }
        ss = warp_sum(ss);
        r = rsqrtf(fmaf(ss, 1.0f / (float)hd, a.eps));
    }
    if (pos < 0) pos = 0;
    if (pos >= a.max_pos) pos = a.max_pos - 1;
    const float* cs = a.cos_t ? a.cos_t + (size_t)pos * half : nullptr;
    const float* sn = a.sin_t ? a.sin_t + (size_t)pos * half : nullptr;
    for (int i = lane; i < half; i += 32) {
        float lo = to_f32(x[i]), hi = to_f32(x[i + half]);
        if (wv) {
            const float wl = a.w_is_f32 ? ((const float*)wv)[i] : to_f32(((const T*)wv)[i]);
            const float wh = a.w_is_f32 ? ((const float*)wv)[i + half] : to_f32(((const T*)wv)[i + half]);
            lo = to_f32(from_f32<T>(lo * r * wl));
            hi = to_f32(from_f32<T>(hi * r * wh));
        }
        if (cs) {
            const float c = cs[i], s = sn[i];
            const float nlo = lo * c - hi * s;
            const float nhi = hi * c + lo * s;
            lo = nlo; hi = nhi;
        }
        const T tlo = from_f32<T>(lo), thi = from_f32<T>(hi);
        x[i] = tlo; x[i + half] = thi;
        if (dst) { dst[i] = tlo; dst[i + half] = thi; }
    }
}

// Two neighbouring elements per lane (4 or 8 bytes per access): the form every model size
// takes whose head size is a multiple of 4 and whose rows start on even elements.
template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<bf16> { using type = __nv_bfloat162; };
__device__ __forceinline__ float2 pair_to_f32(float2 v) { return v; }
__device__ __forceinline__ float2 pair_to_f32(__nv_bfloat162 v) { return __bfloat1622float2(v); }
template <typename T> __device__ __forceinline__ typename Pair<T>::type pair_from_f32(float a, float b);
template <> __device__ __forceinline__ float2 pair_from_f32<float>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 pair_from_f32<bf16>(float a, float b) { return __floats2bfloat162_rn(a, b); }

// Blocks (token, group): the token's position, slot and page are looked up once per block, then
// the block's warps share the heads of its group.  One group per token when there are many tokens
// (the look-up is amortised over all heads), one head per warp when there are few (short chains).
template <typename T>
__global__ void rope_store_pairs_kernel(RopeStoreArgs a) {
    ti_pdl_trigger();
    ti_pdl_sync();
    using P = typename Pair<T>::type;
    const int n_warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_q = a.q ? a.n_heads : 0;
    const int heads_k = a.k ? a.n_kv_heads : 0;
    const int heads_v = a.v ? a.n_kv_heads : 0;
    const int per_tok = heads_q + heads_k + heads_v;
    const int m = blockIdx.x;
    const int hd = a.head_dim, half = hd >> 1;
    int pos = a.tok_pos[m];

    // where the cache keeps this token (head 0 of keys; other heads and values follow from it)
    long long dst_off = -1;
    if (a.k_pages) {
        const int seq = a.tok_seq[m];
        const int slot = a.seq_slot[seq];
        int row = pos;
        bool keep = pos >= 0;
        if (a.ring_rows > 0) {
            keep = keep && pos >= a.seq_len[seq] - a.ring_rows;
            row = pos % a.ring_rows;
        }
        const int pidx = row / a.page_size;
        if (keep && pidx < a.table_width) {
            const int page = a.page_table[(size_t)slot * a.table_width + pidx];
            if (page >= 0 && page < a.n_pages)
                dst_off = ((long long)page * a.n_kv_heads * a.page_size + (row % a.page_size)) * hd;
        }
    }
    if (pos < 0) pos = 0;
    if (pos >= a.max_pos) pos = a.max_pos - 1;
    const float* cs = a.cos_t ? a.cos_t + (size_t)pos * half : nullptr;
    const float* sn = a.sin_t ? a.sin_t + (size_t)pos * half : nullptr;

    for (int item = blockIdx.y * n_warps + warp; item < per_tok; item += n_warps * gridDim.y) {
        int h = item, kind;  // 0 q, 1 k, 2 v
        if (h < heads_q) kind = 0;
        else if (h < heads_q + heads_k) { kind = 1; h -= heads_q; }
        else { kind = 2; h -= heads_q + heads_k; }
        T* x = kind == 0 ? (T*)a.q + (size_t)m * a.q_stride + (size_t)h * hd
             : kind == 1 ? (T*)a.k + (size_t)m * a.k_stride + (size_t)h * hd
                         : (T*)a.v + (size_t)m * a.v_stride + (size_t)h * hd;
        T* dst = nullptr;
        if (kind != 0 && dst_off >= 0)
            dst = (T*)(kind == 1 ? a.k_pages : a.v_pages) + dst_off + (size_t)h * a.page_size * hd;
        if (kind == 2) {
            if (dst)
                for (int i = lane * 2; i < hd; i += 64) *reinterpret_cast<P*>(dst + i) = *reinterpret_cast<const P*>(x + i);
            continue;
        }
        const void* wv = kind == 0 ? a.q_w : a.k_w;
        float r = 1.f;
        if (wv) {
            float ss = 0.f;
            for (int i = lane * 2; i < hd; i += 64) {
                const float2 t = pair_to_f32(*reinterpret_cast<const P*>(x + i));
                ss = fmaf(t.x, t.x, ss);
                ss = fmaf(t.y, t.y, ss);
            }
            ss = warp_sum(ss);
            r = rsqrtf(fmaf(ss, 1.0f / (float)hd, a.eps));
        }
        for (int i = lane * 2; i < half; i += 64) {
            float2 lo = pair_to_f32(*reinterpret_cast<const P*>(x + i));
            float2 hi = pair_to_f32(*reinterpret_cast<const P*>(x + i + half));
            if (wv) {
                float2 wl, wh;
                if (a.w_is_f32) {
                    wl = *reinterpret_cast<const float2*>((const float*)wv + i);
                    wh = *reinterpret_cast<const float2*>((const float*)wv + i + half);
                } else {
                    wl = pair_to_f32(*reinterpret_cast<const P*>((const T*)wv + i));
                    wh = pair_to_f32(*reinterpret_cast<const P*>((const T*)wv + i + half));
                }
                lo.x = to_f32(from_f32<T>(lo.x * r * wl.x)); lo.y = to_f32(from_f32<T>(lo.y * r * wl.y));
                hi.x = to_f32(from_f32<T>(hi.x * r * wh.x)); hi.y = to_f32(from_f32<T>(hi.y * r * wh.y));
            }
            if (cs) {
                const float2 c = *reinterpret_cast<const float2*>(cs + i), sv = *reinterpret_cast<const float2*>(sn + i);
                const float2 nlo = make_float2(lo.x * c.x - hi.x * sv.x, lo.y * c.y - hi.y * sv.y);
                const float2 nhi = make_float2(hi.x * c.x + lo.x * sv.x, hi.y * c.y + lo.y * sv.y);
                lo = nlo; hi = nhi;
            }
            const P plo = pair_from_f32<T>(lo.x, lo.y), phi = pair_from_f32<T>(hi.x, hi.y);
            *reinterpret_cast<P*>(x + i) = plo;
            *reinterpret_cast<P*>(x + i + half) = phi;
            if (dst) { *reinterpret_cast<P*>(dst + i) = plo; *reinterpret_cast<P*>(dst + i + half) = phi; }
        }
    }
}

// bfloat16 heads of 64 or 128 elements with 16-byte aligned rows: a head is shared by hd / 16
// lanes, each with 8 consecutive elements of the lower half and the 8 that pair with them in the
// upper half (two 16-byte loads), so a warp works on four (or eight) heads at once and every
// access is a full 16 bytes.  Same formulas and roundings as the kernels above; this is the form
// that many-token steps run (2,048 tokens of a 4B-shaped layer: 38 us with two-element lanes).
template <int HD>
__global__ void rope_store_vec_kernel(RopeStoreArgs a) {
    ti_pdl_trigger();
    ti_pdl_sync();
    constexpr int LPH = HD / 16, HPW = 32 / LPH, half = HD / 2;
    const int n_warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_q = a.q ? a.n_heads : 0;
    const int heads_k = a.k ? a.n_kv_heads : 0;
    const int heads_v = a.v ? a.n_kv_heads : 0;
    const int per_tok = heads_q + heads_k + heads_v;
    const int m = blockIdx.x;
    int pos = a.tok_pos[m];
    long long dst_off = -1;
    if (a.k_pages) {
        const int seq = a.tok_seq[m];
        const int slot = a.seq_slot[seq];
        int row = pos;
        bool keep = pos >= 0;
        if (a.ring_rows > 0) {
            keep = keep && pos >= a.seq_len[seq] - a.ring_rows;
            row = pos % a.ring_rows;
        }
        const int pidx = row / a.page_size;
        if (keep && pidx < a.table_width) {
            const int page = a.page_table[(size_t)slot * a.table_width + pidx];
            if (page >= 0 && page < a.n_pages)
                dst_off = ((long long)page * a.n_kv_heads * a.page_size + (row % a.page_size)) * HD;
        }
    }
    if (pos < 0) pos = 0;
    if (pos >= a.max_pos) pos = a.max_pos - 1;
    const int sub = lane % LPH, i = sub * 8;
    float c[8] = {}, sn[8] = {};
    if (a.cos_t) tirope::load_angles(a.cos_t + (size_t)pos * half, a.sin_t + (size_t)pos * half, i, c, sn);
    for (int item0 = (blockIdx.y * n_warps + warp) * HPW; item0 < per_tok; item0 += n_warps * gridDim.y * HPW) {
        const int item = item0 + lane / LPH;
        const bool active = item < per_tok;
        int h = active ? item : 0, kind;  // 0 q, 1 k, 2 v
        if (h < heads_q) kind = 0;
        else if (h < heads_q + heads_k) { kind = 1; h -= heads_q; }
        else { kind = 2; h -= heads_q + heads_k; }
        bf16* x = kind == 0 ? (bf16*)a.q + (size_t)m * a.q_stride + (size_t)h * HD
                : kind == 1 ? (bf16*)a.k + (size_t)m * a.k_stride + (size_t)h * HD
                            : (bf16*)a.v + (size_t)m * a.v_stride + (size_t)h * HD;
        bf16* dst = nullptr;
        if (kind != 0 && dst_off >= 0)
            dst = (bf16*)(kind == 1 ? a.k_pages : a.v_pages) + dst_off + (size_t)h * a.page_size * HD;
        uint4 vlo = make_uint4(0, 0, 0, 0), vhi = vlo;
        if (active) {
            vlo = *reinterpret_cast<const uint4*>(x + i);
            vhi = *reinterpret_cast<const uint4*>(x + i + half);
        }
        const bool apply = active && kind != 2;
        tirope::norm_rotate<HD>(vlo, vhi, apply, kind == 0 ? a.q_w : a.k_w, a.w_is_f32, a.eps, a.cos_t != nullptr, c, sn, i);
        if (apply) {
            *reinterpret_cast<uint4*>(x + i) = vlo;
            *reinterpret_cast<uint4*>(x + i + half) = vhi;
        }
        if (active && dst) {
            *reinterpret_cast<uint4*>(dst + i) = vlo;
            *reinterpret_cast<uint4*>(dst + i + half) = vhi;
        }
    }
}

extern "C" int ti_qk_norm_rope_store(
    void* q, void* k, void* v, long long q_stride, long long k_stride, long long v_stride,
    int n_heads, int n_kv_heads, int head_dim,
    const void* q_w, const void* k_w, int w_is_f32, float eps,
    const float* cos_t, const float* sin_t, int rot_dim, int max_pos,
    const int* tok_pos, const int* tok_seq, const int* seq_slot, const int* seq_len,
    void* k_pages, void* v_pages, const int* page_table, int table_width, int page_size,
    int ring_rows, int n_pages, int M, int dtype, cudaStream_t stream) {
    if (M == 0) return 0;
    TI_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "qk_norm_rope_store: head size %d must be even", head_dim);
    TI_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "qk_norm_rope_store: cos and sin tables go together");
    TI_REQUIRE(!cos_t || rot_dim == head_dim,
               "qk_norm_rope_store: rotation over %d of %d elements is not implemented (the whole head only)",
               rot_dim, head_dim);
    TI_REQUIRE(!cos_t || max_pos > 0, "qk_norm_rope_store: empty rotary tables");
    TI_REQUIRE((k_pages == nullptr) == (v_pages == nullptr), "qk_norm_rope_store: k and v pages go together");
    TI_REQUIRE(!k_pages || (page_table && page_size > 0 && table_width > 0 && n_pages > 0 && tok_seq && seq_slot),
               "qk_norm_rope_store: incomplete cache description");
    TI_REQUIRE(ring_rows == 0 || (ring_rows % page_size == 0 && seq_len),
               "qk_norm_rope_store: ring of %d rows is not a multiple of the page size %d", ring_rows, page_size);
    RopeStoreArgs a;
    a.q = q; a.k = k; a.v = k_pages ? v : nullptr;   // values are only ever copied to the cache
    a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim;
    a.q_w = q_w; a.k_w = k_w; a.w_is_f32 = w_is_f32; a.eps = eps;
    a.cos_t = cos_t; a.sin_t = sin_t; a.max_pos = max_pos > 0 ? max_pos : 1;
    a.tok_pos = tok_pos; a.tok_seq = tok_seq; a.seq_slot = seq_slot; a.seq_len = seq_len;
    a.k_pages = k_pages; a.v_pages = v_pages; a.page_table = page_table; a.table_width = table_width;
    a.page_size = page_size; a.ring_rows = ring_rows; a.n_pages = n_pages; a.M = M;
    const int per_tok = (a.q ? n_heads : 0) + (a.k ? n_kv_heads : 0) + (a.v ? n_kv_heads : 0);
    if (per_tok == 0) return 0;
    const long long items = (long long)M * per_tok;
    const int warps = 4;
    const long long blocks = (items + warps - 1) / warps;
    TI_REQUIRE(blocks < 2147483647LL, "qk_norm_rope_store: too many heads x tokens (%lld)", items);
    return ti_dispatch_dtype(dtype, [&](auto t) -> int {
        using T = decltype(t);
        const size_t esz = sizeof(T) * 2;
        auto even = [&](const void* p, long long stride) { return !p || ((reinterpret_cast<uintptr_t>(p) % esz) == 0 && stride % 2 == 0); };
        const bool pairs = head_dim % 4 == 0 && even(q, q_stride) && even(k, k_stride) && even(v, v_stride) &&
                           even(q_w, 0) && even(k_w, 0) && even(k_pages, 0) && even(v_pages, 0) &&
                           (reinterpret_cast<uintptr_t>(cos_t) % 8 == 0) && (reinterpret_cast<uintptr_t>(sin_t) % 8 == 0);
        auto al16 = [&](const void* p, long long stride) { return !p || ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && stride % 8 == 0); };
        const bool vec = std::is_same<T, bf16>::value && (head_dim == 64 || head_dim == 128) && al16(q, q_stride) &&
                         al16(k, k_stride) && al16(v, v_stride) && al16(q_w, 0) && al16(k_w, 0) && al16(k_pages, 0) &&
                         al16(v_pages, 0) && al16(cos_t, 0) && al16(sin_t, 0);
        if (vec) {
            const int w = 4;
            const int hpw = 32 / (head_dim / 16);
            const int need = (per_tok + hpw - 1) / hpw;                 // warp-rounds per token
            const int groups = M >= 1024 ? 1 : (need + w - 1) / w;
            if (head_dim == 128)
                TI_CUDA(ti_launch_class<2>(rope_store_vec_kernel<128>, dim3((unsigned)M, (unsigned)groups), dim3(w * 32), 0, stream, a));
            else
                TI_CUDA(ti_launch_class<2>(rope_store_vec_kernel<64>, dim3((unsigned)M, (unsigned)groups), dim3(w * 32), 0, stream, a));
        }
        else if (pairs) {
            const int w = 4;
            const int groups = M >= 1024 ? 1 : (per_tok + w - 1) / w;
            TI_CUDA(ti_launch_class<2>(rope_store_pairs_kernel<T>, dim3((unsigned)M, (unsigned)groups), dim3(w * 32), 0, stream, a));
        }
        else
            TI_CUDA(ti_launch_class<2>(rope_store_kernel<T>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, a));
        TI_CHECK_LAUNCH("qk_norm_rope_store");
        return 0;
    });
}

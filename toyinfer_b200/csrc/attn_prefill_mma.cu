// Causal grouped-query attention of the tokens of one step, bfloat16, tensor cores, tiles
// brought in by TMA.  Same contract, formulas and two forms as attn_prefill_simt.cu (reference:
// src/prefill.cu:224-379): sequences that start at position 0 (the kernel the bfloat16 engine runs
// prompts of head size 64 with), and, PAGED, new tokens after `seq_start[b]` positions kept in the
// paged cache.  In the second form a block first walks the sequence's pages below the start (a page
// is 64 positions x head_dim of one kv head, one tile) and then the step's own keys and values;
// one online softmax runs over both.
//
// Grid (heads, sequences, query tiles of 64 taken from the last to the first), 128 threads,
// two blocks per SM.  q, k and v are strided views of the projection's output
// [tokens, heads * head_dim]; tensor maps with the 128-byte swizzle cut 64 x 64 boxes out of
// them.  The query tile is loaded once; key/value tiles of 64 positions run through a ring
// of stages guarded by mbarriers, one thread issuing loads ahead.  Key tiles that the causal
// mask or the window excludes entirely are never loaded.
//
// Each warp owns 16 queries: S = Q K^T (mma.m16n8k16), scale, mask, online softmax with the
// running maximum subtracted before every exp, O += P V with P rounded to bfloat16, and
// O / sum at the end.
#include "mma_utils.cuh"
#include "tma.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace {
constexpr int BQ = 64, BKV = 64, THREADS = 128, STAGES = 2;

__device__ __forceinline__ float ex2(float x) {      // 2^x, the hardware's approximation (2 ulp)
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct PrefillArgs {
    const int* cu_new; int n_heads, n_kv_heads; float scale; int window;
    void* out; long long o_stride;
    // PAGED form: where the positions before the step's tokens are kept
    const int* seq_start; const int* seq_slot; const int* page_table; int table_width, ring_rows, n_pages;
};

template <int HD, bool PAGED>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_mma_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap kp_map,
                        const __grid_constant__ CUtensorMap vp_map, PrefillArgs a, int* status) {
    ti_pdl_trigger();
    constexpr int TILE_BYTES = BKV * HD * 2;
    constexpr int KSTEPS = HD / 16, NT = HD / 8;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = smem;                         // [64][HD] swizzled
    unsigned char* kv_s = smem + TILE_BYTES;           // STAGES x (K tile, V tile)
    __shared__ uint64_t full[STAGES], q_full;
    __shared__ int s_abort;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(&full[s], 1);
        mbar_init(&q_full, 1);
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    ti_pdl_sync();      // everything above touched only this block's shared memory

    // Blocks are handed out with x running fastest, then y, then z: the heads are x, the sequences y
    // and the query tiles, from the last to the first, z, so that the long rows of the causal
    // triangle of every head and every sequence start before any short one (with the tiles as x a
    // head's short rows started before the next head's long ones, and the last heads' long rows
    // ended the kernel alone: 2,048 tokens of 32 heads took 71 us where the work, evenly spread,
    // takes 41).  A sequence shorter than the longest has nothing at the highest tile numbers.
    const int b = blockIdx.y, h = blockIdx.x;
    const int tok0 = a.cu_new[b];
    const int n = a.cu_new[b + 1] - tok0;
    const int q0 = ((int)gridDim.z - 1 - (int)blockIdx.z) * BQ;
    if (q0 >= n) return;
    const int kvh = h / (a.n_heads / a.n_kv_heads);
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

    // The step's own keys, counted from the sequence's first new token: tiles kt_lo .. kt_hi.
    const int last_q = min(q0 + BQ, n) - 1;
    const int kt_lo = a.window > 0 ? max(0, q0 - a.window + 1) / BKV : 0;
    const int kt_hi = last_q / BKV;
    // PAGED: the sequence's positions below `start`, one page a tile, pages pt_lo .. pt_lo + n_old - 1,
    // before the step's own.  lo_blk is the oldest position any query of this block reads.
    const int start = PAGED ? a.seq_start[b] : 0;
    const int slot = PAGED ? a.seq_slot[b] : 0;
    const int lo_blk = (PAGED && a.window > 0) ? max(0, start + q0 - a.window + 1) : 0;
    const int pt_lo = lo_blk / BKV;
    const int n_old = (PAGED && lo_blk < start) ? (start - 1) / BKV - pt_lo + 1 : 0;
    const int n_tiles = n_old + kt_hi - kt_lo + 1;

    auto issue = [&](int i) {
        unsigned char* dst = kv_s + (size_t)(i % STAGES) * 2 * TILE_BYTES;
        uint64_t* bar = &full[i % STAGES];
        mbar_expect_tx(bar, 2 * TILE_BYTES);
        if (PAGED && i < n_old) {
            const int p0 = (pt_lo + i) * BKV;
            const int row0 = a.ring_rows > 0 ? p0 % a.ring_rows : p0;
            const int pidx = row0 / BKV;
            int page = pidx < a.table_width ? a.page_table[(size_t)slot * a.table_width + pidx] : 0;
            if (page < 0 || page >= a.n_pages) page = 0;
            const int y = (page * a.n_kv_heads + kvh) * BKV;
#pragma unroll
            for (int bx = 0; bx < HD / 64; bx++) {
                tma_load_2d(dst + bx * (BKV * 128), &kp_map, bx * 64, y, bar);
                tma_load_2d(dst + TILE_BYTES + bx * (BKV * 128), &vp_map, bx * 64, y, bar);
            }
            return;
        }
        const int y = tok0 + (kt_lo + i - n_old) * BKV;
#pragma unroll
        for (int bx = 0; bx < HD / 64; bx++) {
            tma_load_2d(dst + bx * (BKV * 128), &k_map, kvh * HD + bx * 64, y, bar);
            tma_load_2d(dst + TILE_BYTES + bx * (BKV * 128), &v_map, kvh * HD + bx * 64, y, bar);
        }
    };
    if (t == 0) {
        mbar_expect_tx(&q_full, TILE_BYTES);
#pragma unroll
        for (int bx = 0; bx < HD / 64; bx++) tma_load_2d(q_s + bx * (BQ * 128), &q_map, h * HD + bx * 64, tok0 + q0, &q_full);
        for (int i = 0; i < STAGES - 1 && i < n_tiles; i++) issue(i);
    }

    // the warp's 16 queries as A fragments
    uint32_t qf[KSTEPS][4];
    {
        const bool ok = mbar_wait(&q_full, 0);
        if (!ok) { ti_report(status, TI_STATUS_TMA_WAIT); s_abort = 1; }
        __syncthreads();
        if (s_abort) {
            if (t == 0)
                for (int j = 0; j < n_tiles && j < STAGES - 1; j++) mbar_wait(&full[j % STAGES], 0);
            return;
        }
        const int mid = lane >> 3, rr = lane & 7;
        const int row = warp * 16 + (mid & 1) * 8 + rr;
        const uint32_t qb = smem_u32(q_s);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++)
            ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], qb + swizzled_offset<BQ>(row, ks * 16 + (mid >> 1) * 8));
    }
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int qi0 = q0 + warp * 16 + (lane >> 2);       // this thread's rows: qi0 and qi0 + 8
    // scores in base-2 units: exp(x * scale - m) = 2^(x * scale * log2(e) - m2)
    const float scale2 = a.scale * 1.4426950408889634f;

    for (int i = 0; i < n_tiles; i++) {
        const int stage = i % STAGES;
        if (t == 0 && i + STAGES - 1 < n_tiles) issue(i + STAGES - 1);
        if (!mbar_wait(&full[stage], (uint32_t)((i / STAGES) & 1))) {
            // the data never came: note it, work on whatever the buffer holds (shared memory only)
            // and leave at the barrier below, where every thread sees the flag
            ti_report(status, TI_STATUS_TMA_WAIT);
            s_abort = 1;
        }
        const uint32_t kb = smem_u32(kv_s + (size_t)stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        // Key positions are counted from the step's first token of this sequence: a page of older
        // positions starts at a negative k0.  `limit` is where the tile's valid keys end.
        const bool old = PAGED && i < n_old;
        const int k0 = old ? (pt_lo + i) * BKV - start : (kt_lo + i - n_old) * BKV;
        const int limit = old ? 0 : n;
        bool patched = false;
        if (old ? (k0 + BKV > 0 || k0 + start < lo_blk) : (k0 + BKV > n)) {
            // Lines of a page outside [lo_blk, start) may hold anything (this step's tokens, an
            // older turn of the ring, a former owner's), and the rows after a sequence's last new
            // token are another sequence's or nobody's: their value rows are cleared, so that a
            // probability of zero times whatever stands there cannot make a NaN
            unsigned char* vt = kv_s + (size_t)stage * 2 * TILE_BYTES + TILE_BYTES;
            for (int r = warp; r < BKV; r += THREADS / 32) {
                const int p = k0 + start + r;
                if (old ? (p < lo_blk || p >= start) : (k0 + r >= n))
                    for (int d = lane * 8; d < HD; d += 256)
                        *reinterpret_cast<uint4*>(vt + swizzled_offset<BKV>(r, d)) = make_uint4(0, 0, 0, 0);
            }
            patched = true;
            __syncthreads();
        }

        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        {
            const int mid = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++)
#pragma unroll
                for (int np = 0; np < 4; np++) {        // two n-tiles (16 keys) per ldmatrix
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, kb + swizzled_offset<BKV>(np * 16 + (mid >> 1) * 8 + rr, ks * 16 + (mid & 1) * 8));
                    mma_bf16(s[np * 2], qf[ks], b0, b1);
                    mma_bf16(s[np * 2 + 1], qf[ks], b2, b3);
                }
        }
        // scale and mask
        const bool edge = a.window > 0 || k0 + BKV - 1 > q0 + warp * 16 || k0 + BKV > limit;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = s[nt][e] * scale2;
                if (edge) {
                    const int kj = k0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int qi = qi0 + (e >> 1) * 8;
                    const bool ok = kj <= qi && kj < limit && (a.window <= 0 || kj > qi - a.window);
                    v = ok ? v : -INFINITY;
                }
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            alpha[r] = (m_new > -INFINITY && m_new != m_run[r]) ? ex2(m_run[r] - m_new) : 1.f;
            m_run[r] = m_new;
        }
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = m_run[e >> 1] > -INFINITY ? ex2(s[nt][e] - m_run[e >> 1]) : 0.f;
                s[nt][e] = p;
                ls[e >> 1] += p;
            }
        l_run[0] = l_run[0] * alpha[0] + ls[0];
        l_run[1] = l_run[1] * alpha[1] + ls[1];
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {     // some row's maximum moved
#pragma unroll
            for (int i2 = 0; i2 < NT; i2++) { o[i2][0] *= alpha[0]; o[i2][1] *= alpha[0]; o[i2][2] *= alpha[1]; o[i2][3] *= alpha[1]; }
        }
        // O += P V, 16 keys at a time
        {
            const int mid = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < NT / 2; n2++) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, vb + swizzled_offset<BKV>(kk * 16 + (mid & 1) * 8 + rr, n2 * 16 + (mid >> 1) * 8));
                    mma_bf16(o[n2 * 2], pf, b0, b1);
                    mma_bf16(o[n2 * 2 + 1], pf, b2, b3);
                }
            }
        }
        if (patched) fence_proxy_async();   // this stage was written by threads; a TMA load will overwrite it
        __syncthreads();    // the stage may be refilled
        if (s_abort) {
            if (t == 0)
                for (int j = i + 1; j < n_tiles && j < i + STAGES; j++) mbar_wait(&full[j % STAGES], (uint32_t)((j / STAGES) & 1));
            return;
        }
    }

    // normalise and store
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    bf16* out = (bf16*)a.out;
    const int c = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        if (qi0 < n)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + qi0) * a.o_stride + (size_t)h * HD + nt * 8 + c) =
                pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
        if (qi0 + 8 < n)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + qi0 + 8) * a.o_stride + (size_t)h * HD + nt * 8 + c) =
                pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
    }
}

struct MapKey {
    const void* ptr; long long rows, cols, stride;
    bool operator<(const MapKey& o) const { return std::tie(ptr, rows, cols, stride) < std::tie(o.ptr, o.rows, o.cols, o.stride); }
};
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_lock;

int view_map(const void* ptr, long long rows, long long cols, long long stride, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_lock);
    MapKey key{ptr, rows, cols, stride};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        CUtensorMap m;
        if (int rc = ti_make_tensor_map_2d_bf16(&m, ptr, (uint64_t)rows, (uint64_t)cols, (uint64_t)stride * 2, 64, 64)) return rc;
        if (g_maps.size() > 8192) g_maps.clear();
        it = g_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

template <int HD, bool PAGED>
int launch(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const CUtensorMap& kpm, const CUtensorMap& vpm,
           const PrefillArgs& a, int n_seq, int max_new, cudaStream_t stream) {
    constexpr size_t smem = (size_t)BKV * HD * 2 * (1 + 2 * STAGES) + 1024;
    static bool configured = false;
    if (!configured) {
        TI_CUDA(cudaFuncSetAttribute(attn_prefill_mma_kernel<HD, PAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    int* status = ti_status_ptr();
    TI_REQUIRE(status != nullptr, "attention_prefill: no status word");
    dim3 grid(a.n_heads, n_seq, (max_new + BQ - 1) / BQ);
    TI_CUDA(ti_launch(attn_prefill_mma_kernel<HD, PAGED>, grid, dim3(THREADS), smem, stream, qm, km, vm, kpm, vpm, a, status));
    TI_CHECK_LAUNCH(PAGED ? "attention_chunk (tensor cores)" : "attention_prefill (tensor cores)");
    return 0;
}

int check_and_map(const char* what, const void* q, const void* k, const void* v, const void* out, long long q_stride,
                  long long k_stride, long long v_stride, long long o_stride, int n_seq, int n_tokens, int n_heads,
                  int n_kv_heads, int head_dim, CUtensorMap* qm, CUtensorMap* km, CUtensorMap* vm) {
    TI_REQUIRE(head_dim == 64 || head_dim == 128, "%s (tensor cores): head size %d is not 64 or 128", what, head_dim);
    TI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "%s: bad head counts", what);
    TI_REQUIRE(n_seq <= 65535 && n_heads <= 65535, "%s: too many sequences or heads for one launch", what);
    TI_REQUIRE(n_tokens <= 65535 * BQ, "%s: %d tokens are too many for one launch", what, n_tokens);
    TI_REQUIRE(q_stride % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0 && o_stride % 2 == 0,
               "%s (tensor cores): token strides must be multiples of 8 elements", what);
    TI_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(out) & 3) == 0, "%s (tensor cores): misaligned operands", what);
    if (int rc = view_map(q, n_tokens, (long long)n_heads * head_dim, q_stride, qm)) return rc;
    if (int rc = view_map(k, n_tokens, (long long)n_kv_heads * head_dim, k_stride, km)) return rc;
    if (int rc = view_map(v, n_tokens, (long long)n_kv_heads * head_dim, v_stride, vm)) return rc;
    return 0;
}
}  // namespace

// bfloat16 only; head_dim 64 or 128.  n_tokens is the number of rows of q, k and v.
extern "C" int ti_attn_prefill_mma(const void* q, const void* k, const void* v, void* out,
                                   long long q_stride, long long k_stride, long long v_stride, long long o_stride,
                                   const int* cu_new, int n_seq, int max_new, int n_tokens, int n_heads, int n_kv_heads,
                                   int head_dim, float scale, int window, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    CUtensorMap qm, km, vm;
    if (int rc = check_and_map("attention_prefill", q, k, v, out, q_stride, k_stride, v_stride, o_stride, n_seq, n_tokens,
                               n_heads, n_kv_heads, head_dim, &qm, &km, &vm)) return rc;
    PrefillArgs a = {};
    a.cu_new = cu_new; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.scale = scale; a.window = window;
    a.out = out; a.o_stride = o_stride;
    return head_dim == 64 ? launch<64, false>(qm, km, vm, km, vm, a, n_seq, max_new, stream)
                          : launch<128, false>(qm, km, vm, km, vm, a, n_seq, max_new, stream);
}

// The same for new tokens after `seq_start[b]` positions that the cache holds (pages of 64
// positions, bfloat16); arguments as ti_attn_chunk_simt.
extern "C" int ti_attn_chunk_mma(const void* q, const void* k, const void* v, void* out,
                                 long long q_stride, long long k_stride, long long v_stride, long long o_stride,
                                 const int* cu_new, const int* seq_start, const int* seq_slot, int n_seq, int max_new,
                                 int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                 const void* k_pages, const void* v_pages, const int* page_table, int table_width,
                                 int page_size, int ring_rows, int n_pages, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(k_pages && v_pages && page_table && seq_start && seq_slot && table_width > 0 && n_pages > 0,
               "attention_chunk: incomplete cache description");
    TI_REQUIRE(page_size == BKV, "attention_chunk (tensor cores): pages of %d positions, this kernel works on %d", page_size, BKV);
    TI_REQUIRE(ring_rows % page_size == 0, "attention_chunk: ring of %d rows is not whole pages", ring_rows);
    TI_REQUIRE(ring_rows == 0 || (window > 0 && ring_rows >= window),
               "attention_chunk: a ring of %d rows needs a window of at most as many positions (got %d)", ring_rows, window);
    TI_REQUIRE(((reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) == 0,
               "attention_chunk (tensor cores): cache pages must be 16-byte aligned");
    CUtensorMap qm, km, vm, kpm, vpm;
    if (int rc = check_and_map("attention_chunk", q, k, v, out, q_stride, k_stride, v_stride, o_stride, n_seq, n_tokens,
                               n_heads, n_kv_heads, head_dim, &qm, &km, &vm)) return rc;
    const long long rows = (long long)n_pages * n_kv_heads * BKV;
    if (int rc = view_map(k_pages, rows, head_dim, head_dim, &kpm)) return rc;
    if (int rc = view_map(v_pages, rows, head_dim, head_dim, &vpm)) return rc;
    PrefillArgs a = {};
    a.cu_new = cu_new; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.scale = scale; a.window = window;
    a.out = out; a.o_stride = o_stride;
    a.seq_start = seq_start; a.seq_slot = seq_slot; a.page_table = page_table; a.table_width = table_width;
    a.ring_rows = ring_rows; a.n_pages = n_pages;
    return head_dim == 64 ? launch<64, true>(qm, km, vm, kpm, vpm, a, n_seq, max_new, stream)
                          : launch<128, true>(qm, km, vm, kpm, vpm, a, n_seq, max_new, stream);
}

// Grouped-query attention of one new token per sequence over the paged cache, bfloat16,
// tensor cores, keys and values brought in by TMA.  Same contract and formulas as
// attn_decode_simt.cu (reference: src/decode.cu:401-432, :471-532, :598-628); this is the
// kernel the bfloat16 engine decodes with for head sizes 64 and 128.
//
// Grid (sequences, kv heads x groups of 16 query heads, splits), 128 threads, up to two
// blocks per SM.  The cache page of a tile (64 positions x head_dim of one kv head, 8 or
// 16 KB, contiguous) arrives as 64x64 boxes through a tensor map with the 128-byte
// swizzle, into a ring of STAGES buffers guarded by mbarriers; one thread issues the loads
// STAGES-1 tiles ahead.  The step is bound by the read of the cache: every key and value
// byte is read once for all query heads of its kv head.
//
// Each warp owns 16 of a tile's 64 positions and keeps an online softmax of its own:
//   S = Q K^T   mma.m16n8k16, the query heads (padded to 16 rows) as the M dimension,
//   P = exp(S * scale - max), O += P V with P rounded to bfloat16 for the second product.
// The four warps' maxima, sums and outputs are merged through shared memory at the end,
// then written as this split's partial result (or the final one when there is one split).
//
// With CLUSTER the blocks of a sequence's kv head (its splits, up to 16) are launched as one
// thread-block cluster and merge their partial results themselves, through distributed shared
// memory: every block leaves its merged partial in its own shared memory, a cluster barrier makes
// them visible, and each block then forms a slice of the final outputs from all blocks' partials
// (read with ld.shared::cluster, added in split order).  No partial result goes through global
// memory and no second kernel runs.
#include "attn_decode.cuh"
#include "mma_utils.cuh"
#include "rope_math.cuh"
#include "tcgen05.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace {
constexpr int TILE = 64, THREADS = 128, STAGES = 3;

template <int HD>
__device__ __forceinline__ uint32_t tile_offset(int row, int d) { return swizzled_offset<TILE>(row, d); }

__device__ __forceinline__ float ex2(float x) {      // 2^x, the hardware's approximation (2 ulp)
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The new token's projections as the product before this kernel left them: not yet normed,
// rotated or stored.  With FUSED the kernel does that itself (formulas and rounding as in
// rope_store.cu: per-head RMS norm rounded to bfloat16, then the rotation of pairs i, i + hd/2,
// rounded again), so that one kernel fewer stands between the projection and the attention.
// k and v are null for a layer that reads another layer's memory.
struct FuseArgs {
    const bf16* q; const bf16* k; const bf16* v;        // [B, heads, hd], [B, kv_heads, hd] twice
    long long q_stride, k_stride, v_stride;             // elements between consecutive sequences
    const void* q_w; const void* k_w; int w_is_f32; float eps;   // norm weights [hd] or null
    const float* cos_t; const float* sin_t; int max_pos;         // rotary tables [max_pos, hd/2] or null
    bf16* k_pages; bf16* v_pages;                       // the cache, writable
};

__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_address) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_address) : "memory");
    return v;
}

template <int HD, bool FUSED, bool CLUSTER>
__global__ void __launch_bounds__(THREADS, 2)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                       tiattn::DecodeArgs a, FuseArgs f, int* status) {
    ti_pdl_trigger();
    constexpr int TILE_BYTES = TILE * HD * 2;          // one of K or V
    constexpr int KSTEPS = HD / 16, NT = HD / 8;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of the boxes is what the swizzle pattern is defined against
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[STAGES];
    __shared__ int s_abort;
    __shared__ __align__(16) bf16 q_s[FUSED ? 16 * HD : 8];       // the block's query heads, normed and rotated
    __shared__ __align__(16) bf16 kv_new[FUSED ? 2 * HD : 8];     // the new token's key and value of this kv head

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(&full[s], 1);
        // once a wait has run out somewhere results are lost anyway: later blocks leave at once
        s_abort = *reinterpret_cast<volatile int*>(status);
        mbar_fence_init();
    }
    __syncthreads();
    // (in a cluster every block goes on to the cluster's two barriers: it does no work, and the
    // other blocks, which read the same word sooner or later, report what they see themselves)
    const bool dead = s_abort != 0;
    if (dead && !CLUSTER) return;

    // What is read before ti_pdl_sync() below does not depend on the kernel just before this
    // one: the step's lengths, slots and page table were uploaded before the step's first
    // kernel, and cache lines of positions before the newest were written in earlier steps.
    const int b = blockIdx.x, split = blockIdx.z;
    const int g = a.n_heads / a.n_kv_heads;
    const int groups = (g + 15) / 16;
    const int kvh = blockIdx.y / groups, grp = blockIdx.y - kvh * groups;
    const int h0 = kvh * g + grp * 16;                 // first query head of this block
    const int rows = min(16, g - grp * 16);            // query heads of this block
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int L = a.seq_len[b];
    const int slot = a.seq_slot[b];
    const int lo = a.window > 0 ? max(0, L - a.window) : 0;
    const int tile_lo = lo / TILE;
    const int n_tiles = L > 0 ? (L - 1) / TILE - tile_lo + 1 : 0;
    const int per = (n_tiles + a.n_splits - 1) / a.n_splits;
    const int my_lo = tile_lo + split * per;
    const int my_n = dead ? 0 : max(0, min(my_lo + per, tile_lo + n_tiles) - my_lo);

    auto issue = [&](int i) {      // tile my_lo + i into stage i % STAGES; one thread calls this
        const int p0 = (my_lo + i) * TILE;
        const int row0 = a.ring_rows > 0 ? p0 % a.ring_rows : p0;
        const int pidx = row0 / TILE;
        int page = pidx < a.table_width ? a.page_table[(size_t)slot * a.table_width + pidx] : 0;
        if (page < 0 || page >= a.n_pages) page = 0;
        const int y = (page * a.n_kv_heads + kvh) * TILE;
        unsigned char* dst = smem + (size_t)(i % STAGES) * 2 * TILE_BYTES;
        uint64_t* bar = &full[i % STAGES];
        mbar_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
        for (int bx = 0; bx < HD / 64; bx++) {
            tma_load_2d(dst + bx * (TILE * 128), &k_map, bx * 64, y, bar);
            tma_load_2d(dst + TILE_BYTES + bx * (TILE * 128), &v_map, bx * 64, y, bar);
        }
    };
    // The tile that holds the newest position is being written by the kernel before this one;
    // every other tile may be requested right away, while that kernel still runs.
    // (With FUSED nobody writes the cache before this kernel does: every tile may come early; the
    // newest position's line is put into the tile by hand below.)
    const int newest_tile = (L - 1) / TILE;
    unsigned early = 0;
    if (t == 0)
        for (int i = 0; i < STAGES - 1 && i < my_n; i++)
            if (FUSED || my_lo + i != newest_tile) { issue(i); early |= 1u << i; }
    ti_pdl_sync();
    if (t == 0)
        for (int i = 0; i < STAGES - 1 && i < my_n; i++)
            if (!((early >> i) & 1u)) issue(i);

    const bool store_new = FUSED && f.k != nullptr;
    const bool has_newest = L > 0 && newest_tile >= my_lo && newest_tile < my_lo + my_n;
    if (FUSED) {
        const bf16* fq = ti_dependent(f.q);
        const bf16* fk = ti_dependent(f.k);
        const bf16* fv = ti_dependent(f.v);
        int pos = max(L - 1, 0);
        if (pos >= f.max_pos) pos = f.max_pos - 1;
        // heads of this block's queries, then the kv head's key and value: hd / 16 lanes a head
        constexpr int LPH = HD / 16, HPW = 32 / LPH;
        const int sub = lane % LPH, ei = sub * 8;
        float c[8] = {}, sn[8] = {};
        if (f.cos_t) tirope::load_angles(f.cos_t + (size_t)pos * (HD / 2), f.sin_t + (size_t)pos * (HD / 2), ei, c, sn);
        const int n_items = rows + (store_new ? 2 : 0);
        for (int item0 = warp * HPW; item0 < n_items; item0 += (THREADS / 32) * HPW) {
            const int item = item0 + lane / LPH;
            const bool active = item < n_items;
            const bool is_q = item < rows, is_v = item == rows + 1;
            const bf16* src = is_q ? fq + (size_t)b * f.q_stride + (size_t)(h0 + item) * HD
                            : !is_v ? fk + (size_t)b * f.k_stride + (size_t)kvh * HD
                                    : fv + (size_t)b * f.v_stride + (size_t)kvh * HD;
            bf16* dst = is_q ? q_s + item * HD : kv_new + (is_v ? HD : 0);
            uint4 vlo = make_uint4(0, 0, 0, 0), vhi = vlo;
            if (active) {
                vlo = *reinterpret_cast<const uint4*>(src + ei);
                vhi = *reinterpret_cast<const uint4*>(src + ei + HD / 2);
            }
            tirope::norm_rotate<HD>(vlo, vhi, active && !is_v, is_q ? f.q_w : f.k_w, f.w_is_f32, f.eps, f.cos_t != nullptr, c, sn, ei);
            if (active) {
                *reinterpret_cast<uint4*>(dst + ei) = vlo;
                *reinterpret_cast<uint4*>(dst + ei + HD / 2) = vhi;
            }
        }
        __syncthreads();
        // the new key and value go to their line of the cache, for the steps to come: one block per
        // (sequence, kv head) does it, the one whose tiles include the newest position
        if (store_new && has_newest && grp == 0 && t < 2 * (HD / 8)) {
            const int row = a.ring_rows > 0 ? (L - 1) % a.ring_rows : L - 1;
            const int pidx = row / TILE;
            const int page = pidx < a.table_width ? a.page_table[(size_t)slot * a.table_width + pidx] : -1;
            if (page >= 0 && page < a.n_pages) {
                const bool is_v = t >= HD / 8;
                const int c = (is_v ? t - HD / 8 : t) * 8;
                bf16* dst = (is_v ? f.v_pages : f.k_pages) + (((size_t)page * a.n_kv_heads + kvh) * TILE + row % TILE) * HD + c;
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(kv_new + (is_v ? HD : 0) + c);
            }
        }
    }
    // the queries as A fragments: row lane/4 (and +8) is a query head, zero beyond `rows`
    uint32_t qf[KSTEPS][4];
    {
        const bf16* q = FUSED ? q_s : (const bf16*)a.q + (size_t)b * a.q_stride + (size_t)h0 * HD;
        const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            const int d = ks * 16 + c;
            qf[ks][0] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q + (size_t)r0 * HD + d) : 0u;
            qf[ks][1] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q + (size_t)r1 * HD + d) : 0u;
            qf[ks][2] = r0 < rows ? *reinterpret_cast<const uint32_t*>(q + (size_t)r0 * HD + d + 8) : 0u;
            qf[ks][3] = r1 < rows ? *reinterpret_cast<const uint32_t*>(q + (size_t)r1 * HD + d + 8) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows lane/4 and lane/4 + 8

    // Scores are kept in base-2 units: exp(x * scale - m) = 2^(x * scale * log2(e) - m2), one
    // multiply-add and one ex2 per element.
    const float scale2 = a.scale * 1.4426950408889634f;
    const bool upper = rows > 8;        // rows lane/4 + 8 are real query heads, not padding
    for (int i = 0; i < my_n; i++) {
        const int stage = i % STAGES;
        if (t == 0 && i + STAGES - 1 < my_n) issue(i + STAGES - 1);   // its stage was drained in iteration i-1
        if (!mbar_wait(&full[stage], (uint32_t)((i / STAGES) & 1))) {
            // the data never came: note it, work on whatever the buffer holds (shared memory only)
            // and leave at the barrier below, where every thread sees the flag
            ti_report(status, TI_STATUS_TMA_WAIT);
            s_abort = 1;
        }
        const uint32_t kbase = smem_u32(smem + (size_t)stage * 2 * TILE_BYTES);
        const uint32_t vbase = kbase + TILE_BYTES;
        const int p0 = (my_lo + i) * TILE;
        const int key0 = warp * 16;                      // this warp's positions within the tile
        const bool patched = store_new && my_lo + i == newest_tile;
        const bool edge = p0 < lo || p0 + TILE > L || patched;      // some positions of the tile are out of range (or written by hand)
        if (patched) {
            // the newest position's key and value are not in the cache the tile was read from
            const int rr = (L - 1) - p0;
            if (warp == rr / 16 && lane < 2 * (HD / 8)) {
                const bool is_v = lane >= HD / 8;
                const int c = (is_v ? lane - HD / 8 : lane) * 8;
                *reinterpret_cast<uint4*>(smem + (size_t)stage * 2 * TILE_BYTES + (is_v ? TILE_BYTES : 0) + tile_offset<HD>(rr, c)) =
                    *reinterpret_cast<const uint4*>(kv_new + (is_v ? HD : 0) + c);
            }
            __syncwarp();
        }

        if (edge) {
            // lines outside [lo, L) may hold anything: clear this warp's such value rows
            for (int r = 0; r < 16; r++) {
                const int p = p0 + key0 + r;
                if (p < lo || p >= L)
                    for (int d = lane * 8; d < HD; d += 256)
                        *reinterpret_cast<uint4*>(smem + (size_t)stage * 2 * TILE_BYTES + TILE_BYTES + tile_offset<HD>(key0 + r, d)) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }

        // S = Q K^T for 16 positions: two n-tiles of 8, even and odd K steps summed separately
        // so that four chains of dependent MMAs run instead of two
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            const int mid = lane >> 3, rr = lane & 7;
            const int key = key0 + (mid >> 1) * 8 + rr;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks += 2) {
                uint32_t b0, b1, b2, b3, c0, c1, c2, c3;
                ldmatrix_x4(b0, b1, b2, b3, kbase + tile_offset<HD>(key, ks * 16 + (mid & 1) * 8));
                ldmatrix_x4(c0, c1, c2, c3, kbase + tile_offset<HD>(key, (ks + 1) * 16 + (mid & 1) * 8));
                mma_bf16(s[0], qf[ks], b0, b1);
                mma_bf16(s[1], qf[ks], b2, b3);
                mma_bf16(s2[0], qf[ks + 1], c0, c1);
                mma_bf16(s2[1], qf[ks + 1], c2, c3);
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) s[nt][e] += s2[nt][e];
        }
        // scale, mask, online softmax (rows lane/4 and lane/4 + 8; columns are positions)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int p = p0 + key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                const bool ok = !edge || (p >= lo && p < L);
                s[nt][e] = ok ? s[nt][e] * scale2 : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
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
        uint32_t pf[4];
        {
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                p[nt][0] = m_run[0] > -INFINITY ? ex2(s[nt][0] - m_run[0]) : 0.f;
                p[nt][1] = m_run[0] > -INFINITY ? ex2(s[nt][1] - m_run[0]) : 0.f;
                p[nt][2] = (upper && m_run[1] > -INFINITY) ? ex2(s[nt][2] - m_run[1]) : 0.f;
                p[nt][3] = (upper && m_run[1] > -INFINITY) ? ex2(s[nt][3] - m_run[1]) : 0.f;
            }
            l_run[0] = l_run[0] * alpha[0] + p[0][0] + p[0][1] + p[1][0] + p[1][1];   // this thread's share of the row
            l_run[1] = l_run[1] * alpha[1] + p[0][2] + p[0][3] + p[1][2] + p[1][3];
            pf[0] = pack_bf16(p[0][0], p[0][1]);
            pf[1] = pack_bf16(p[0][2], p[0][3]);
            pf[2] = pack_bf16(p[1][0], p[1][1]);
            pf[3] = pack_bf16(p[1][2], p[1][3]);
        }
        // O = O * alpha + P V; the rescaling is skipped while no row's maximum moved
        {
            const bool rescale = __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f);
            const int mid = lane >> 3, rr = lane & 7;
            const int key = key0 + (mid & 1) * 8 + rr;
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; n2++) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, vbase + tile_offset<HD>(key, n2 * 16 + (mid >> 1) * 8));
                if (rescale) {
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        float(&acc)[4] = o[n2 * 2 + h];
                        acc[0] *= alpha[0]; acc[1] *= alpha[0]; acc[2] *= alpha[1]; acc[3] *= alpha[1];
                    }
                }
                mma_bf16(o[n2 * 2], pf, b0, b1);
                mma_bf16(o[n2 * 2 + 1], pf, b2, b3);
            }
        }
        if (edge) fence_proxy_async();   // this stage was written by threads; a TMA load will overwrite it
        __syncthreads();                 // the stage may be refilled
        if (s_abort) {
            // give the loads still in flight a bounded time to land before the block's shared
            // memory is released (or used for the merge), then leave without a result
            if (t == 0)
                for (int j = i + 1; j < my_n && j < i + STAGES; j++) mbar_wait(&full[j % STAGES], (uint32_t)((j / STAGES) & 1));
            if (!CLUSTER) return;
            break;
        }
    }
    // back to natural-log units for the merge
#pragma unroll
    for (int r = 0; r < 2; r++) m_run[r] *= 0.6931471805599453f;

    // ---- merge the four warps (each holds an online softmax over its own positions)
    __syncthreads();
    float* Om = reinterpret_cast<float*>(smem);            // [4 warps][16 rows][HD]
    float* Mm = Om + 4 * 16 * HD;                          // [4][16]
    float* Lm = Mm + 4 * 16;                               // [4][16]
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < NT; n++) {
            float* w0 = Om + ((size_t)warp * 16 + r0) * HD + n * 8 + c;
            float* w1 = Om + ((size_t)warp * 16 + r0 + 8) * HD + n * 8 + c;
            w0[0] = o[n][0]; w0[1] = o[n][1];
            w1[0] = o[n][2]; w1[1] = o[n][3];
        }
        if ((lane & 3) == 0) {
            Mm[warp * 16 + r0] = m_run[0]; Mm[warp * 16 + r0 + 8] = m_run[1];
            Lm[warp * 16 + r0] = l_run[0]; Lm[warp * 16 + r0 + 8] = l_run[1];
        }
    }
    __syncthreads();
    float* fin_o = Lm + 4 * 16;                            // CLUSTER: this block's merged partial, [16 rows][HD]
    float* fin_ml = fin_o + 16 * HD;                       //          and its (maximum, sum) per row
    for (int idx = t; idx < rows * HD; idx += THREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) m = fmaxf(m, Mm[w * 16 + r]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float mw = Mm[w * 16 + r];
            if (mw > -INFINITY) {
                const float f = expf(mw - m);
                l += Lm[w * 16 + r] * f;
                acc += Om[((size_t)w * 16 + r) * HD + d] * f;
            }
        }
        const int h = h0 + r;
        if (CLUSTER) {
            fin_o[idx] = acc;
            if (d == 0) { fin_ml[r * 2] = m; fin_ml[r * 2 + 1] = l; }
        } else if (a.n_splits == 1) {
            ((bf16*)a.out)[(size_t)b * a.o_stride + (size_t)h * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            const size_t base = ((size_t)b * a.n_heads + h) * a.n_splits + split;
            a.part_o[base * HD + d] = acc;
            if (d == 0) { a.part_ml[base * 2] = m; a.part_ml[base * 2 + 1] = l; }
        }
    }
    if (CLUSTER) {
        // every block's partial is in its shared memory: make them visible to the cluster, then
        // each block forms its slice of the outputs from all of them, in split order
        cluster_sync_all();
        const int total = rows * HD, n = a.n_splits;
        const int share = (total + n - 1) / n;
        const int lo_idx = (int)cluster_rank() * share, hi_idx = min(total, lo_idx + share);
        for (int idx = lo_idx + t; idx < hi_idx; idx += THREADS) {
            const int r = idx / HD, d = idx - r * HD;
            float m = -INFINITY;
            for (int sp = 0; sp < n; sp++) m = fmaxf(m, ld_cluster_f32(cluster_addr(&fin_ml[r * 2], (uint32_t)sp)));
            float l = 0.f, acc = 0.f;
            for (int sp = 0; sp < n; sp++) {
                const float ms = ld_cluster_f32(cluster_addr(&fin_ml[r * 2], (uint32_t)sp));
                if (ms > -INFINITY) {       // a split that saw no key contributes nothing
                    const float w = expf(ms - m);
                    l = fmaf(ld_cluster_f32(cluster_addr(&fin_ml[r * 2 + 1], (uint32_t)sp)), w, l);
                    acc = fmaf(ld_cluster_f32(cluster_addr(&fin_o[idx], (uint32_t)sp)), w, acc);
                }
            }
            ((bf16*)a.out)[(size_t)b * a.o_stride + (size_t)(h0 + r) * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        }
        cluster_sync_all();     // nobody leaves while its shared memory may still be read
    }
}

struct MapKey {
    const void* ptr; long long rows; int hd;
    bool operator<(const MapKey& o) const { return std::tie(ptr, rows, hd) < std::tie(o.ptr, o.rows, o.hd); }
};
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_maps_lock;

int page_map(const void* pages, long long rows, int hd, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_maps_lock);
    MapKey key{pages, rows, hd};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        CUtensorMap m;
        if (int rc = ti_make_tensor_map_2d_bf16(&m, pages, (uint64_t)rows, (uint64_t)hd, (uint64_t)hd * 2, TILE, 64)) return rc;
        if (g_maps.size() > 4096) g_maps.clear();
        it = g_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

constexpr int MAX_CLUSTER = 16;      // blocks of one cluster; above 8 the kernel must opt in (non-portable size)

// mode: 0 partial results through global memory and a combine kernel started like every kernel,
// 1 the same with the combine kernel started late, 2 the splits as one cluster that merges itself.
template <int HD, bool FUSED>
int launch(const tiattn::DecodeArgs& a, const FuseArgs& f, int n_seq, int mode, cudaStream_t stream) {
    constexpr size_t stage_bytes = 2 * TILE * HD * 2;
    constexpr size_t merge_bytes = (4 * 16 * HD + 2 * 4 * 16 + 16 * HD + 2 * 16) * sizeof(float);
    constexpr size_t smem = (STAGES * stage_bytes > merge_bytes ? STAGES * stage_bytes : merge_bytes) + 1024;
    static bool configured = false;
    if (!configured) {
        TI_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel<HD, FUSED, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TI_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel<HD, FUSED, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TI_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel<HD, FUSED, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        configured = true;
    }
    CUtensorMap km, vm;
    const long long rows = (long long)a.n_pages * a.n_kv_heads * TILE;
    if (int rc = page_map(a.k_pages, rows, HD, &km)) return rc;
    if (int rc = page_map(a.v_pages, rows, HD, &vm)) return rc;
    int* status = ti_status_ptr();
    TI_REQUIRE(status != nullptr, "attention_decode: no status word");
    const int g = a.n_heads / a.n_kv_heads;
    dim3 grid(n_seq, a.n_kv_heads * ((g + 15) / 16), a.n_splits);
    if (mode == 2) {
        TI_REQUIRE(a.n_splits >= 2 && a.n_splits <= MAX_CLUSTER, "attention_decode (cluster): %d splits do not form a cluster of 2 to %d blocks",
                   a.n_splits, MAX_CLUSTER);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        int n_attr = 0;
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = (unsigned)a.n_splits;
        n_attr++;
        if (ti_pdl_enabled(3)) {
            attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
            n_attr++;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        TI_CUDA(cudaLaunchKernelEx(&cfg, attn_decode_mma_kernel<HD, FUSED, true>, km, vm, a, f, status));
        TI_CHECK_LAUNCH("attention_decode (tensor cores, cluster)");
        return 0;
    }
    TI_CUDA(ti_launch_class<3>(attn_decode_mma_kernel<HD, FUSED, false>, grid, dim3(THREADS), smem, stream, km, vm, a, f, status));
    TI_CHECK_LAUNCH("attention_decode (tensor cores)");
    if (a.n_splits > 1) {
        dim3 cgrid(n_seq, a.n_heads);
        // Started late when the caller says so: by then the attention blocks with their large shared
        // memory are gone and the SMs have drained, so that few-token products after it find an L1
        // (see gemm_skinny.cu) and may start early.  Before the tcgen05 product (more tokens), which
        // does not care about L1 and gains from starting early, it starts early like everything else.
        if (mode == 1)
            TI_CUDA(ti_launch_after(tiattn::attn_decode_combine_kernel<bf16>, cgrid, dim3(HD < 128 ? 64 : 128), 0, stream, (const float*)a.part_o, (const float*)a.part_ml, (bf16*)a.out, a.o_stride, a.n_heads, HD, a.n_splits));
        else
            TI_CUDA(ti_launch_class<4>(tiattn::attn_decode_combine_kernel<bf16>, cgrid, dim3(HD < 128 ? 64 : 128), 0, stream, (const float*)a.part_o, (const float*)a.part_ml, (bf16*)a.out, a.o_stride, a.n_heads, HD, a.n_splits));
        TI_CHECK_LAUNCH("attention_decode (combine)");
    }
    return 0;
}
}  // namespace

namespace {
template <int HD, bool FUSED>
int cluster_room(int n_splits, int* room) {
    constexpr size_t stage_bytes = 2 * TILE * HD * 2;
    constexpr size_t merge_bytes = (4 * 16 * HD + 2 * 4 * 16 + 16 * HD + 2 * 16) * sizeof(float);
    constexpr size_t smem = (STAGES * stage_bytes > merge_bytes ? STAGES * stage_bytes : merge_bytes) + 1024;
    TI_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel<HD, FUSED, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    TI_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel<HD, FUSED, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, n_splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)n_splits;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TI_CUDA(cudaOccupancyMaxActiveClusters(room, attn_decode_mma_kernel<HD, FUSED, true>, &cfg));
    return 0;
}
}  // namespace

// How many clusters of n_splits blocks of the cluster form of the kernel the device holds at once
// (0: such a cluster cannot be placed at all).  The host merges through a cluster only when all
// clusters of a step find room together: a second round of clusters costs more than the merge
// through global memory saves.
extern "C" int ti_attn_decode_cluster_room(int head_dim, int fused, int n_splits, int* room) {
    TI_REQUIRE(head_dim == 64 || head_dim == 128, "attention_decode (cluster): head size %d is not 64 or 128", head_dim);
    TI_REQUIRE(n_splits >= 1 && n_splits <= MAX_CLUSTER && room != nullptr, "attention_decode (cluster): bad cluster size %d", n_splits);
    if (head_dim == 64) return fused ? cluster_room<64, true>(n_splits, room) : cluster_room<64, false>(n_splits, room);
    return fused ? cluster_room<128, true>(n_splits, room) : cluster_room<128, false>(n_splits, room);
}

// bfloat16 only; head_dim 64 or 128; pages of 64 positions.  Same arguments as
// ti_attn_decode_simt, plus `mode`: how the splits' results are merged (see launch above; with
// mode 2 no scratch is needed).
extern "C" int ti_attn_decode_mma(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                  const int* page_table, int table_width, int page_size, int ring_rows,
                                  int n_pages, const int* seq_slot, const int* seq_len, int n_seq,
                                  int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                  int n_splits, void* out, long long o_stride, float* part_o,
                                  float* part_ml, int dtype, int mode, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(dtype == TI_BF16, "attention_decode (tensor cores): bfloat16 only");
    TI_REQUIRE(head_dim == 64 || head_dim == 128, "attention_decode (tensor cores): head size %d is not 64 or 128", head_dim);
    TI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention_decode: bad head counts");
    TI_REQUIRE(page_size == TILE, "attention_decode: pages of %d positions, this kernel works on %d", page_size, TILE);
    TI_REQUIRE(ring_rows % page_size == 0, "attention_decode: ring of %d rows is not whole pages", ring_rows);
    TI_REQUIRE(window == 0 || ring_rows == 0 || ring_rows >= window, "attention_decode: ring smaller than the window");
    TI_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention_decode: bad split count %d", n_splits);
    TI_REQUIRE(n_splits == 1 || mode == 2 || (part_o && part_ml), "attention_decode: split results need scratch memory");
    TI_REQUIRE((reinterpret_cast<uintptr_t>(q) & 3) == 0 && q_stride % 2 == 0, "attention_decode: queries must be 4-byte aligned");
    tiattn::DecodeArgs a;
    a.q = q; a.q_stride = q_stride; a.k_pages = k_pages; a.v_pages = v_pages; a.page_table = page_table;
    a.table_width = table_width; a.page_size = page_size; a.ring_rows = ring_rows; a.n_pages = n_pages;
    a.seq_slot = seq_slot; a.seq_len = seq_len; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim;
    a.window = window; a.n_splits = n_splits; a.scale = scale; a.out = out; a.o_stride = o_stride;
    a.part_o = part_o; a.part_ml = part_ml;
    FuseArgs f = {};
    return head_dim == 64 ? launch<64, false>(a, f, n_seq, mode, stream) : launch<128, false>(a, f, n_seq, mode, stream);
}

// The same with the step before it folded in: q[B, heads, hd], k and v[B, kv_heads, hd] are the
// projection's output for the one new token of each sequence (position seq_len - 1).  Per head:
// RMS norm with q_w / k_w (null: none; float32 or bfloat16), rotation by the float32 tables
// cos, sin [max_pos, hd/2] (null: none), then k and v are written to their line of the cache and
// the attention runs.  k and v null: a layer that reads another's memory; only q is prepared.
extern "C" int ti_attn_decode_fused(const void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                    long long v_stride, const void* q_w, const void* k_w, int w_is_f32, float eps,
                                    const float* cos_t, const float* sin_t, int max_pos,
                                    void* k_pages, void* v_pages, const int* page_table, int table_width, int page_size,
                                    int ring_rows, int n_pages, const int* seq_slot, const int* seq_len, int n_seq,
                                    int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                    void* out, long long o_stride, float* part_o, float* part_ml, int dtype,
                                    int mode, cudaStream_t stream) {
    if (n_seq == 0) return 0;
    TI_REQUIRE(dtype == TI_BF16, "attention_decode (fused): bfloat16 only");
    TI_REQUIRE(head_dim == 64 || head_dim == 128, "attention_decode (fused): head size %d is not 64 or 128", head_dim);
    TI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention_decode: bad head counts");
    TI_REQUIRE(page_size == TILE, "attention_decode: pages of %d positions, this kernel works on %d", page_size, TILE);
    TI_REQUIRE(ring_rows % page_size == 0, "attention_decode: ring of %d rows is not whole pages", ring_rows);
    TI_REQUIRE(window == 0 || ring_rows == 0 || ring_rows >= window, "attention_decode: ring smaller than the window");
    TI_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention_decode: bad split count %d", n_splits);
    TI_REQUIRE(n_splits == 1 || mode == 2 || (part_o && part_ml), "attention_decode: split results need scratch memory");
    TI_REQUIRE(q != nullptr && (k == nullptr) == (v == nullptr), "attention_decode (fused): queries are needed; keys and values go together");
    TI_REQUIRE((cos_t == nullptr) == (sin_t == nullptr) && (!cos_t || max_pos > 0), "attention_decode (fused): cos and sin tables go together");
    auto ok16 = [](const void* p, long long stride) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && stride % 8 == 0; };
    TI_REQUIRE(ok16(q, q_stride) && ok16(k, k_stride) && ok16(v, v_stride) && ok16(q_w, 0) && ok16(k_w, 0) && ok16(cos_t, 0) && ok16(sin_t, 0),
               "attention_decode (fused): projections, norm weights and rotary tables must be 16-byte aligned, strides multiples of 8");
    TI_REQUIRE((reinterpret_cast<uintptr_t>(k_pages) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_pages) & 15) == 0,
               "attention_decode (fused): cache pages must be 16-byte aligned");
    tiattn::DecodeArgs a;
    a.q = q; a.q_stride = q_stride; a.k_pages = k_pages; a.v_pages = v_pages; a.page_table = page_table;
    a.table_width = table_width; a.page_size = page_size; a.ring_rows = ring_rows; a.n_pages = n_pages;
    a.seq_slot = seq_slot; a.seq_len = seq_len; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.hd = head_dim;
    a.window = window; a.n_splits = n_splits; a.scale = scale; a.out = out; a.o_stride = o_stride;
    a.part_o = part_o; a.part_ml = part_ml;
    FuseArgs f;
    f.q = (const bf16*)q; f.k = (const bf16*)k; f.v = (const bf16*)v;
    f.q_stride = q_stride; f.k_stride = k_stride; f.v_stride = v_stride;
    f.q_w = q_w; f.k_w = k_w; f.w_is_f32 = w_is_f32; f.eps = eps;
    f.cos_t = cos_t; f.sin_t = sin_t; f.max_pos = max_pos > 0 ? max_pos : 1;
    f.k_pages = (bf16*)k_pages; f.v_pages = (bf16*)v_pages;
    return head_dim == 64 ? launch<64, true>(a, f, n_seq, mode, stream) : launch<128, true>(a, f, n_seq, mode, stream);
}

// Causal grouped-query attention over the tokens of one step on the 5th-generation tensor
// cores: both products of a tile, S = Q K^T and O += P V, are tcgen05 MMAs with their
// accumulators in tensor memory.  Same contract and formulas as attn_prefill_simt.cu
// (reference: src/prefill.cu:224-379); head_dim 64 or 128, bfloat16.  Two forms, as there: sequences
// that start at position 0, and, PAGED, new tokens after `seq_start[b]` positions kept in the
// paged cache: a block then first walks the sequence's pages below the start (a page is 64
// positions x head_dim of one kv head: one key tile and one value tile, read with the same TMA
// box as a tile of the step) and then the step's own keys and values; one online softmax runs
// over both, and nothing but the source of a tile's loads and its mask knows the difference.
//
// A block owns 128 queries of one head (grid: heads, sequences, query tiles from the last to
// the first) and walks over key/value tiles of 64 positions; tiles that the causal mask or the
// window excludes entirely are never loaded.  Roles, 320 threads:
//   warp 0     TMA: the query tile once, then key tiles and value tiles, each into a ring of two
//              buffers of its own: a key buffer is free as soon as the first product has read it, so
//              the next keys arrive while the softmax of this tile runs;
//   warp 1     one lane issues the MMAs: S_{j+1} = Q K_{j+1}^T goes out before O += P_j V_j, into
//              the other of two score buffers in tensor memory, so the tensor cores work on the
//              next tile's scores while the softmax warps are busy with this tile's.  Descriptors
//              are made once: this thread's chain of instructions and waits sets the block's pace;
//   warps 2-9  softmax: two threads per query row (= TMEM lane), 32 of the tile's 64 positions each;
//              warps w and w + 4 share a quarter of the lanes.  A thread reads its scores once,
//              the halves exchange the row maximum through shared memory, and P = 2^(s - m) goes
//              back as bfloat16 into tensor memory over the scores (the second MMA takes its A
//              operand from there).  The warps are bound by the number of instructions they issue:
//              scale and subtraction are one packed float32 multiply-add per two scores, sums are
//              packed adds, maxima three-input.
// Measured with clock64 stamps per tile (one block, 2,048 tokens): the loop TMA -> first product ->
// softmax -> second product -> buffer free took 2,400 cycles per tile with one ring for keys and
// values and one thread per row, 1,770 with this arrangement, of which the issuing thread is busy
// about 1,400 and a tile's softmax takes about 1,400.
// The output accumulator stays in tensor memory for the whole row of tiles.  It is rescaled
// only when a row's maximum has grown by more than 2^8 since the scale was last fixed (P then
// holds values up to 256 instead of 1, which float32 sums and bfloat16 products carry without
// loss); the final division by the running sum makes the result the same.
// V is stored [position][d]: for the second product that is the "MN-major" form of the B
// operand, described as such to the MMA instead of being transposed.
#include "tcgen05.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace {
constexpr int BQ = 128, BKV = 64, THREADS = 320;      // TMA warp, MMA warp, eight softmax warps

struct Args {
    const int* cu_new; int n_heads, n_kv_heads; float scale; int window;
    void* out; long long o_stride;
    // PAGED form: where the positions before the step's tokens are kept
    const int* seq_start; const int* seq_slot; const int* page_table; int table_width, ring_rows, n_pages;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two floats in one 64-bit register pair, for the packed float32 instructions of sm_100: the
// softmax warps are bound by how many instructions they issue, and these do two elements each.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Shared memory of a block (all dynamic, so that two blocks fit an SM): the query tile, two
// stages of (K tile, V tile), then the mbarriers.
template <int HD> struct Smem {
    static constexpr int Q_BYTES = BQ * HD * 2, KV_BYTES = BKV * HD * 2;
    static constexpr int Q_OFF = 0, KV_OFF = Q_BYTES, BAR_OFF = KV_OFF + 4 * KV_BYTES;
    static constexpr int MX_OFF = BAR_OFF + 256;          // row maxima of the two column halves, two tiles deep
    static constexpr int L_OFF = MX_OFF + 2 * 2 * BQ * 4;  // row sums of the two column halves
    static constexpr int TOTAL = L_OFF + 2 * BQ * 4;
};

template <int HD, bool PAGED>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                       const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap kp_map,
                       const __grid_constant__ CUtensorMap vp_map, Args a, int* status) {
    ti_pdl_trigger();
    using L = Smem<HD>;
    constexpr int Q_BYTES = L::Q_BYTES, KV_BYTES = L::KV_BYTES;
    constexpr int QBOX = 128 * 128, KBOX = BKV * 128;      // bytes of one 64-column box of 128 / BKV rows
    constexpr uint32_t S_COLS = BKV, O_COL = 2 * BKV;      // tensor memory: S0 | S1 | O
    constexpr uint32_t TMEM_COLS = 256;
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* q_s = smem + L::Q_OFF;
    unsigned char* kv_s = smem + L::KV_OFF;                // stage s: K at kv_s + s * 2 * KV_BYTES, V after it
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;      // [2]
    uint64_t* v_full = bars + 3;      // [2]
    uint64_t* k_empty = bars + 5;     // [2] a tile's first product has read its keys
    uint64_t* v_empty = bars + 7;     // [2] a tile's second product has read its values
    uint64_t* s_full = bars + 9;      // [2] scores of a tile are in tensor memory
    uint64_t* p_full = bars + 11;     // [2] the softmax warps have replaced them by P
    uint64_t* pv_done = bars + 13;    //     a tile's second product has finished (one phase per tile)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    int* gave_up = reinterpret_cast<int*>(bars + 16);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Once a wait has run out somewhere, results are lost anyway: later blocks leave at once
    // instead of each running into its own limits (a stuck step then ends in seconds, not minutes).
    if (threadIdx.x == 0) *gave_up = *reinterpret_cast<volatile int*>(status);
    __syncthreads();
    if (*gave_up) return;
    if (smem_u32(smem) & 1023u) {       // the swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0) ti_report(status, TI_STATUS_PIPE_WAIT);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; s++) {
            mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 8);
        }
        mbar_init(pv_done, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        __syncwarp();
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    ti_pdl_sync();

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
    const bool active = q0 < n;
    const int kvh = h / (a.n_heads / a.n_kv_heads);
    const int last_q = min(q0 + BQ, n) - 1;
    const int kt_lo = a.window > 0 ? max(0, q0 - a.window + 1) / BKV : 0;
    // PAGED: the sequence's positions below `start`, one page a tile, pages pt_lo .. pt_lo + n_old - 1,
    // before the step's own.  lo_blk is the oldest position any query of this block reads.  Key
    // positions are counted from the step's first token of the sequence, so a page's are negative.
    const int start = PAGED ? a.seq_start[b] : 0;
    const int slot = PAGED ? a.seq_slot[b] : 0;
    const int lo_blk = (PAGED && a.window > 0) ? max(0, start + q0 - a.window + 1) : 0;
    const int pt_lo = lo_blk / BKV;
    const int n_old = (PAGED && active && lo_blk < start) ? (start - 1) / BKV - pt_lo + 1 : 0;
    const int n_tiles = active ? n_old + last_q / BKV - kt_lo + 1 : 0;

    if (active && warp_uniform() == 0) {
        if (elect_one()) {
            mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int bx = 0; bx < HD / 64; bx++) tma_load_2d(q_s + bx * QBOX, &q_map, h * HD + bx * 64, tok0 + q0, q_full);
            // Keys run one tile ahead of values: the keys of tile j + 1 are asked for as soon as the
            // first product of tile j - 1 has read that buffer, the values of tile j once the second
            // product of tile j - 2 has read theirs.
            // the first row, in the tensor map of the pages, of the page that holds tile j of the old positions
            auto page_row = [&](int j) -> int {
                const int p0 = (pt_lo + j) * BKV;
                const int pidx = (a.ring_rows > 0 ? p0 % a.ring_rows : p0) / BKV;
                int page = pidx < a.table_width ? a.page_table[(size_t)slot * a.table_width + pidx] : 0;
                if (page < 0 || page >= a.n_pages) page = 0;
                return (page * a.n_kv_heads + kvh) * BKV;
            };
            auto load_k = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait(&k_empty[s], (uint32_t)(((j >> 1) & 1) ^ 1))) { ti_report(status, TI_STATUS_PIPE_WAIT); return false; }
                unsigned char* ks = kv_s + (size_t)s * 2 * KV_BYTES;
                mbar_expect_tx(&k_full[s], KV_BYTES);
                if (PAGED && j < n_old) {
                    const int y = page_row(j);
#pragma unroll
                    for (int bx = 0; bx < HD / 64; bx++) tma_load_2d(ks + bx * KBOX, &kp_map, bx * 64, y, &k_full[s]);
                    return true;
                }
#pragma unroll
                for (int bx = 0; bx < HD / 64; bx++) tma_load_2d(ks + bx * KBOX, &k_map, kvh * HD + bx * 64, tok0 + (kt_lo + j - n_old) * BKV, &k_full[s]);
                return true;
            };
            auto load_v = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait(&v_empty[s], (uint32_t)(((j >> 1) & 1) ^ 1))) { ti_report(status, TI_STATUS_PIPE_WAIT); return false; }
                unsigned char* vs = kv_s + (size_t)s * 2 * KV_BYTES + KV_BYTES;
                mbar_expect_tx(&v_full[s], KV_BYTES);
                if (PAGED && j < n_old) {
                    const int y = page_row(j);
#pragma unroll
                    for (int bx = 0; bx < HD / 64; bx++) tma_load_2d(vs + bx * KBOX, &vp_map, bx * 64, y, &v_full[s]);
                    return true;
                }
#pragma unroll
                for (int bx = 0; bx < HD / 64; bx++) tma_load_2d(vs + bx * KBOX, &v_map, kvh * HD + bx * 64, tok0 + (kt_lo + j - n_old) * BKV, &v_full[s]);
                return true;
            };
            bool ok = n_tiles > 0 && load_k(0);
            for (int j = 0; j < n_tiles && ok; j++) {
                if (j + 1 < n_tiles) ok = load_k(j + 1);
                if (ok) ok = load_v(j);
            }
        }
    } else if (active && warp_uniform() == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc_s = instr_desc_bf16(BKV, false);    // S: N = positions, K tile K-major
            constexpr uint32_t idesc_o = instr_desc_bf16(HD, true);      // O: N = head elements, V tile MN-major
            // The one thread that issues the products is on the block's critical path: descriptors
            // are made once; inside the loop a descriptor is a base plus a constant (the address
            // field counts 16-byte units and cannot overflow within shared memory).
            const uint64_t q_desc = smem_desc_sw128(smem_u32(q_s));
            const uint64_t k_desc0 = smem_desc_sw128(smem_u32(kv_s)), k_desc1 = smem_desc_sw128(smem_u32(kv_s + 2 * KV_BYTES));
            const uint64_t v_desc0 = smem_desc_mn_sw128(smem_u32(kv_s + KV_BYTES), KBOX);
            const uint64_t v_desc1 = smem_desc_mn_sw128(smem_u32(kv_s + 3 * KV_BYTES), KBOX);
            auto issue_s = [&](int j) {       // S_j = Q K_j^T into score buffer j & 1
                const uint64_t kd = (j & 1) ? k_desc1 : k_desc0;
                const uint32_t d = tmem + (j & 1) * S_COLS;
#pragma unroll
                for (int kk = 0; kk < HD / 16; kk++)      // 64 columns per box, 32 bytes per step of 16
                    tc_mma_bf16(d, q_desc + (uint64_t)(((kk >> 2) * QBOX + (kk & 3) * 32) >> 4),
                                kd + (uint64_t)(((kk >> 2) * KBOX + (kk & 3) * 32) >> 4), idesc_s, kk > 0 ? 1u : 0u);
                tc_commit(&s_full[j & 1]);
                tc_commit(&k_empty[j & 1]);      // the keys have been read once these products are through
            };
            bool ok = mbar_wait(q_full, 0) && mbar_wait(&k_full[0], 0);
            if (!ok) ti_report(status, TI_STATUS_TMA_WAIT);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < n_tiles && ok; j++) {
                if (j + 1 < n_tiles) {
                    // its score buffer holds P of tile j-1: that tile's second product must have read it.
                    // (Products of different accumulators are not promised to run in the order of issue,
                    // so the wait stays although this thread issued that product first.)
                    const int sb = (j + 1) & 1, u = (j + 1) >> 1;
                    if (!mbar_wait(&k_full[sb], (uint32_t)(u & 1)) || (j > 0 && !mbar_wait(pv_done, (uint32_t)((j - 1) & 1)))) {
                        ti_report(status, TI_STATUS_TMA_WAIT); ok = false; break;
                    }
                    tc_fence_after();
                    issue_s(j + 1);
                }
                if (!mbar_wait(&p_full[j & 1], (uint32_t)((j >> 1) & 1)) || !mbar_wait(&v_full[j & 1], (uint32_t)((j >> 1) & 1))) {
                    ti_report(status, TI_STATUS_PIPE_WAIT); ok = false; break;
                }
                tc_fence_after();
                const uint64_t vd = (j & 1) ? v_desc1 : v_desc0;
                const uint32_t p_tmem = tmem + (j & 1) * S_COLS;       // P: two bfloat16 per column, 8 columns per step
#pragma unroll
                for (int kk = 0; kk < BKV / 16; kk++)        // 16 positions per step
                    tc_mma_bf16_ts(tmem + O_COL, p_tmem + kk * 8, vd + (uint64_t)((kk * 16 * 128) >> 4),
                                   idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(&v_empty[j & 1]);      // the values have been read
                tc_commit(pv_done);              // and O holds this tile's contribution
            }
        }
    } else if (active) {
        // ---- softmax: two threads per query row (= TMEM lane), each with 32 of the tile's 64
        // positions.  Warps 2-5 take the first 32 columns, warps 6-9 the second; warp w and w + 4
        // share the lanes 32 * (w % 4) .. + 31, the quarter of tensor memory a warp may touch.
        // The halves meet once per tile, for the row maximum (shared memory, a barrier of their
        // own); sums stay apart until the end.  A thread that saw a wait run out keeps going
        // through the barriers without touching anything, so that nobody is left waiting for it.
        const int qd = warp & 3, half = (warp - 2) >> 2;
        const int r = qd * 32 + lane;
        const int qi = q0 + r;
        const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
        const float scale2 = a.scale * 1.4426950408889634f;
        float* mx_s = reinterpret_cast<float*>(smem + L::MX_OFF);      // [tile parity][half][row]
        float* l_s = reinterpret_cast<float*>(smem + L::L_OFF);        // [half][row]
        constexpr int HALF = BKV / 2;
        float m_used = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; j++) {
            const int sb = j & 1;
            if (ok && !mbar_wait(&s_full[sb], (uint32_t)((j >> 1) & 1))) { ti_report(status, TI_STATUS_MMA_WAIT); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            const bool old = PAGED && j < n_old;
            const int tile0 = old ? (pt_lo + j) * BKV - start : (kt_lo + j - n_old) * BKV;   // the tile's first position
            const int limit = old ? 0 : n;                                                  // where its valid keys end
            const int k0 = tile0 + half * HALF;
            const bool edge = a.window > 0 || k0 + HALF - 1 > q0 + qd * 32 || k0 + HALF > limit;
            const uint32_t s_addr = tmem + sb * S_COLS + lane_base;
            // this thread's 32 scores of the row, as the product left them (the scale comes later)
            float v[HALF];
            if (ok) {
                tmem_ld32(s_addr + half * HALF, v);
            } else {
#pragma unroll
                for (int e = 0; e < HALF; e++) v[e] = -INFINITY;
            }
            if (edge) {
#pragma unroll
                for (int e = 0; e < HALF; e++) {
                    const int kj = k0 + e;
                    const bool vis = kj <= qi && kj < limit && (a.window <= 0 || kj > qi - a.window);
                    v[e] = vis ? v[e] : -INFINITY;
                }
            }
            // row maximum in base-2 units (the scale is positive): three-input maxima, four chains
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < HALF; e += 8) {
                mx4[0] = max3(mx4[0], v[e], v[e + 1]); mx4[1] = max3(mx4[1], v[e + 2], v[e + 3]);
                mx4[2] = max3(mx4[2], v[e + 4], v[e + 5]); mx4[3] = max3(mx4[3], v[e + 6], v[e + 7]);
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale2;
            mx_s[(sb * 2 + half) * BQ + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + qd) : "memory");      // the two warps that share these rows
            mx = fmaxf(mx, mx_s[(sb * 2 + (half ^ 1)) * BQ + r]);
            float alpha = 1.f, m_new = m_used;
            if (mx > m_used + 8.f || (m_used == -INFINITY && mx > -INFINITY)) {
                m_new = mx;
                alpha = ex2(m_used - m_new);        // 0 when nothing was visible before
            }
            const float m_sub = m_new > -INFINITY ? m_new : 0.f;      // masked scores stay -inf, 2^-inf = 0
            // p = 2^(s * scale - m): one packed multiply-add per two scores, two exponentials, one
            // packed add into the sums, one conversion to a bfloat16 pair
            const unsigned long long sc2 = pack2(scale2, scale2), nm2 = pack2(-m_sub, -m_sub);
            unsigned long long sum2[2] = {0ull, 0ull};
            uint32_t pk[HALF / 2];
#pragma unroll
            for (int e = 0; e < HALF; e += 4) {
                float x0, x1, x2, x3;
                unpack2(fma2(pack2(v[e], v[e + 1]), sc2, nm2), x0, x1);
                unpack2(fma2(pack2(v[e + 2], v[e + 3]), sc2, nm2), x2, x3);
                const float p0 = ex2(x0), p1 = ex2(x1), p2 = ex2(x2), p3 = ex2(x3);
                sum2[0] = add2(sum2[0], pack2(p0, p1));
                sum2[1] = add2(sum2[1], pack2(p2, p3));
                __nv_bfloat162 t0 = __floats2bfloat162_rn(p0, p1), t1 = __floats2bfloat162_rn(p2, p3);
                pk[e >> 1] = *reinterpret_cast<uint32_t*>(&t0);
                pk[(e >> 1) + 1] = *reinterpret_cast<uint32_t*>(&t1);
            }
            float sum4[4];
            unpack2(sum2[0], sum4[0], sum4[1]);
            unpack2(sum2[1], sum4[2], sum4[3]);
            if (old ? (tile0 + BKV > 0 || tile0 + start < lo_blk) : (tile0 + BKV > n)) {
                // Lines of a page outside [lo_blk, start) may hold anything (this step's tokens, an
                // older turn of the ring, a former owner's), and the rows after a sequence's last new
                // token are another sequence's or nobody's: their value rows are cleared, so that a
                // probability of zero times whatever stands there cannot make a NaN.  A row of a box is
                // 128 bytes whatever the swizzle does inside it; four threads clear a row of all boxes.
                // The second product starts only after every softmax warp has arrived on p_full below,
                // and the next load into this buffer only after that product.
                if (ok && !mbar_wait(&v_full[sb], (uint32_t)((j >> 1) & 1))) { ti_report(status, TI_STATUS_TMA_WAIT); ok = false; }
                if (ok) {
                    const int st = (int)threadIdx.x - 64, row = st >> 2, part = st & 3;
                    const int p = tile0 + start + row;
                    if (old ? (p < lo_blk || p >= start) : (tile0 + row >= n)) {
                        constexpr int PART = HD / 2;        // bytes of a row's HD * 2 that one of its four threads clears
                        uint4* dst = reinterpret_cast<uint4*>(kv_s + (size_t)sb * 2 * KV_BYTES + KV_BYTES + (part * PART / 128) * KBOX +
                                                              row * 128 + (part * PART) % 128);
#pragma unroll
                        for (int e = 0; e < PART / 16; e++) dst[e] = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();
                }
            }
            // Every tile's completion is waited for, in order, before this tile's P is handed over, whether
            // or not O is touched.  (Waiting only when a row rescales looked safe on paper and gave wrong
            // rows now and then at 32 heads and three sequences: tests/test_kernels_gpu.py,
            // test_attention_prefill_tcgen05_at_long_lengths.)
            const bool rescale = j > 0 && __any_sync(0xffffffffu, alpha != 1.f);
            if (ok && j > 0 && !mbar_wait(pv_done, (uint32_t)((j - 1) & 1))) { ti_report(status, TI_STATUS_MMA_WAIT); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                if (rescale) {
                    // Each half rescales its 64 of the row's 128 columns.
                    tc_fence_after();
#pragma unroll 1
                    for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); c++) {
                        float o[32];
                        tmem_ld32(tmem + O_COL + lane_base + c * 32, o);
#pragma unroll
                        for (int e = 0; e < 32; e++) o[e] *= alpha;
                        tmem_st32(tmem + O_COL + lane_base + c * 32, o);
                    }
                }
                // P over the scores: this thread's 32 values as 16 columns of bfloat16 pairs
                tmem_st16_bits(s_addr + half * (HALF / 2), pk);
                l_run = l_run * alpha + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                m_used = m_new;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[sb]);
            }
        }
        if (ok && n_tiles > 0) {
            if (!mbar_wait(pv_done, (uint32_t)((n_tiles - 1) & 1))) { ti_report(status, TI_STATUS_MMA_WAIT); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
        }
        // the row's sum: both halves'
        l_s[half * BQ + r] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + qd) : "memory");      // the two warps that share these rows
        l_run += l_s[(half ^ 1) * BQ + r];
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            bf16* orow = (bf16*)a.out + (size_t)(tok0 + qi) * a.o_stride + (size_t)h * HD;
#pragma unroll 1
            for (int c = half * (HD / 64); c < (half + 1) * (HD / 64); c++) {
                float o[32];
                tmem_ld32(tmem + O_COL + lane_base + c * 32, o);
                if (qi < n) {
                    uint32_t ok4[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        __nv_bfloat162 t = __floats2bfloat162_rn(o[e] * inv, o[e + 1] * inv);
                        ok4[e >> 1] = *reinterpret_cast<uint32_t*>(&t);
                    }
#pragma unroll
                    for (int t4 = 0; t4 < 4; t4++)
                        *reinterpret_cast<uint4*>(orow + c * 32 + t4 * 8) = make_uint4(ok4[t4 * 4], ok4[t4 * 4 + 1], ok4[t4 * 4 + 2], ok4[t4 * 4 + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

struct MapKey {
    const void* ptr; long long rows, cols, stride; int box_rows;
    bool operator<(const MapKey& o) const {
        return std::tie(ptr, rows, cols, stride, box_rows) < std::tie(o.ptr, o.rows, o.cols, o.stride, o.box_rows);
    }
};
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_lock;

int view_map(const void* ptr, long long rows, long long cols, long long stride, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> guard(g_lock);
    MapKey key{ptr, rows, cols, stride, box_rows};
    auto it = g_maps.find(key);
    if (it == g_maps.end()) {
        CUtensorMap m;
        if (int rc = ti_make_tensor_map_2d_bf16(&m, ptr, (uint64_t)rows, (uint64_t)cols, (uint64_t)stride * 2, (uint32_t)box_rows, 64)) return rc;
        if (g_maps.size() > 8192) g_maps.clear();
        it = g_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}
}  // namespace

namespace {
int check_common(const char* what, const void* q, const void* k, const void* v, const void* out, long long q_stride,
                 long long k_stride, long long v_stride, long long o_stride, int n_seq, int n_tokens, int n_heads,
                 int n_kv_heads, int head_dim, CUtensorMap* qm, CUtensorMap* km, CUtensorMap* vm) {
    TI_REQUIRE(head_dim == 64 || head_dim == 128, "%s (tcgen05): head size %d is not 64 or 128", what, head_dim);
    TI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "%s: bad head counts", what);
    TI_REQUIRE(n_seq <= 65535 && n_heads <= 65535, "%s: too many sequences or heads for one launch", what);
    TI_REQUIRE(n_tokens <= 65535 * BQ, "%s: %d tokens are too many for one launch", what, n_tokens);
    TI_REQUIRE(q_stride % 8 == 0 && k_stride % 8 == 0 && v_stride % 8 == 0 && o_stride % 8 == 0,
               "%s (tcgen05): token strides must be multiples of 8 elements", what);
    TI_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                 reinterpret_cast<uintptr_t>(out)) & 15) == 0, "%s (tcgen05): misaligned operands", what);
    if (int rc = view_map(q, n_tokens, (long long)n_heads * head_dim, q_stride, BQ, qm)) return rc;
    if (int rc = view_map(k, n_tokens, (long long)n_kv_heads * head_dim, k_stride, BKV, km)) return rc;
    if (int rc = view_map(v, n_tokens, (long long)n_kv_heads * head_dim, v_stride, BKV, vm)) return rc;
    return 0;
}

template <int HD, bool PAGED>
int launch(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const CUtensorMap& kpm, const CUtensorMap& vpm,
           const Args& a, int n_seq, int max_new, cudaStream_t stream) {
    constexpr size_t smem = Smem<HD>::TOTAL;
    static bool configured = false;
    if (!configured) {
        TI_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<HD, PAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    int* status = ti_status_ptr();
    TI_REQUIRE(status != nullptr, "attention_prefill: no status word");
    dim3 grid(a.n_heads, n_seq, (max_new + BQ - 1) / BQ);
    TI_CUDA(ti_launch(attn_prefill_tc_kernel<HD, PAGED>, grid, dim3(THREADS), smem, stream, qm, km, vm, kpm, vpm, a, status));
    TI_CHECK_LAUNCH(PAGED ? "attention_chunk (tcgen05)" : "attention_prefill (tcgen05)");
    return 0;
}
}  // namespace

// bfloat16, head_dim 64 or 128.  Same arguments as ti_attn_prefill_mma.
extern "C" int ti_attn_prefill_tc(const void* q, const void* k, const void* v, void* out,
                                  long long q_stride, long long k_stride, long long v_stride, long long o_stride,
                                  const int* cu_new, int n_seq, int max_new, int n_tokens, int n_heads, int n_kv_heads,
                                  int head_dim, float scale, int window, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    CUtensorMap qm, km, vm;
    if (int rc = check_common("attention_prefill", q, k, v, out, q_stride, k_stride, v_stride, o_stride, n_seq, n_tokens,
                              n_heads, n_kv_heads, head_dim, &qm, &km, &vm)) return rc;
    Args a = {};
    a.cu_new = cu_new; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.scale = scale; a.window = window;
    a.out = out; a.o_stride = o_stride;
    return head_dim == 64 ? launch<64, false>(qm, km, vm, km, vm, a, n_seq, max_new, stream)
                          : launch<128, false>(qm, km, vm, km, vm, a, n_seq, max_new, stream);
}

// The same for new tokens after `seq_start[b]` positions that the cache holds (pages of 64
// positions, bfloat16); arguments as ti_attn_chunk_mma.
extern "C" int ti_attn_chunk_tc(const void* q, const void* k, const void* v, void* out,
                                long long q_stride, long long k_stride, long long v_stride, long long o_stride,
                                const int* cu_new, const int* seq_start, const int* seq_slot, int n_seq, int max_new,
                                int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                const void* k_pages, const void* v_pages, const int* page_table, int table_width,
                                int page_size, int ring_rows, int n_pages, cudaStream_t stream) {
    if (n_seq == 0 || max_new == 0) return 0;
    TI_REQUIRE(k_pages && v_pages && page_table && seq_start && seq_slot && table_width > 0 && n_pages > 0,
               "attention_chunk: incomplete cache description");
    TI_REQUIRE(page_size == BKV, "attention_chunk (tcgen05): pages of %d positions, this kernel works on %d", page_size, BKV);
    TI_REQUIRE(ring_rows % page_size == 0, "attention_chunk: ring of %d rows is not whole pages", ring_rows);
    TI_REQUIRE(ring_rows == 0 || (window > 0 && ring_rows >= window),
               "attention_chunk: a ring of %d rows needs a window of at most as many positions (got %d)", ring_rows, window);
    TI_REQUIRE(((reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) == 0,
               "attention_chunk (tcgen05): cache pages must be 16-byte aligned");
    CUtensorMap qm, km, vm, kpm, vpm;
    if (int rc = check_common("attention_chunk", q, k, v, out, q_stride, k_stride, v_stride, o_stride, n_seq, n_tokens,
                              n_heads, n_kv_heads, head_dim, &qm, &km, &vm)) return rc;
    const long long rows = (long long)n_pages * n_kv_heads * BKV;
    if (int rc = view_map(k_pages, rows, head_dim, head_dim, BKV, &kpm)) return rc;
    if (int rc = view_map(v_pages, rows, head_dim, head_dim, BKV, &vpm)) return rc;
    Args a = {};
    a.cu_new = cu_new; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.scale = scale; a.window = window;
    a.out = out; a.o_stride = o_stride;
    a.seq_start = seq_start; a.seq_slot = seq_slot; a.page_table = page_table; a.table_width = table_width;
    a.ring_rows = ring_rows; a.n_pages = n_pages;
    return head_dim == 64 ? launch<64, true>(qm, km, vm, kpm, vpm, a, n_seq, max_new, stream)
                          : launch<128, true>(qm, km, vm, kpm, vpm, a, n_seq, max_new, stream);
}

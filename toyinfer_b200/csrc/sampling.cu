// Choosing the next token from float32 logits: argmax, and temperature sampling with
// top-k and top-p.
//
// The reference samples on the CPU (src/sampler.cpp:18-69): greedy when
// |temperature| < 1e-3 or top_k == 1 (first maximum wins, :71-81); otherwise
// x = logit / temperature, the k largest are kept, p = softmax over them, sorted
// descending, the list is cut after the first entry at which the running sum exceeds
// top_p, and a uniform draw times that sum picks the first entry whose running sum
// exceeds it.  It divides by the temperature a second time inside the exponent
// (:38) and seeds its generator from the clock (:57-60); here the temperature
// applies once and the uniform number is a pure function of (seed, sequence key,
// step), so a sequence draws the same numbers in any batch.
//
// One block of 1024 threads per row.  Which of the two rules applies is the host's
// decision.  Three kernels: up to 1,024 candidates (one sort in shared memory), the whole
// vocabulary without limits (one scan), and everything else tier by tier.
#include "common.cuh"

#include <climits>

namespace {
constexpr int SB = 1024;      // threads per block
constexpr int MAXK = 1024;    // candidates the top-k path can sort

__device__ __forceinline__ unsigned order_key(float x) {
    if (x == 0.f) x = 0.f;      // -0 counts as +0, as in a float comparison
    const unsigned u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float <=> larger key
}

// uniform in [0, 1) with 24 bits, from (seed, key, step)
__host__ __device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long key,
                                                       unsigned long long step) {
    unsigned long long x = seed * 0x9E3779B97F4A7C15ull + key * 0xBF58476D1CE4E5B9ull +
                           step * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return (float)(x >> 40) * (1.0f / 16777216.0f);
}

// exclusive prefix sums over the block's threads in thread order; returns the total
template <typename V>
__device__ V block_exclusive_scan(V v, V* total, V* sm /* 33 entries */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    V inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const V n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) sm[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        V w = lane < (blockDim.x >> 5) ? sm[lane] : V(0);
        V winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const V n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        sm[lane] = winc - w;
        if (lane == 31) sm[32] = winc;
    }
    __syncthreads();
    *total = sm[32];
    return sm[warp] + inc - v;
}

// The maximum of a row with its index as one 64-bit word that atomicMax can order: the
// value's order-preserving key above, the index counted down below, so that among equal
// values the lower index is the larger word.  -0 counts as +0, as in a float comparison.
__device__ __forceinline__ unsigned long long pack_best(float v, int i) {
    if (v == 0.f) v = 0.f;
    return ((unsigned long long)order_key(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
}

// Grid (rows, chunks), 256 threads.  Each block finds the first maximum of its chunk and
// folds it into the row's word; the block that arrives last (a ticket per row) writes the
// index and leaves word and ticket zero for the next call.  NaNs are never chosen; a row of
// nothing but NaNs gives index 0.
constexpr int AB = 256;
__global__ void __launch_bounds__(AB) argmax_kernel(const float* __restrict__ logits, long long ld, int V, int per,
                                                    unsigned long long* __restrict__ best_word,
                                                    int* __restrict__ tickets, int* __restrict__ out) {
    ti_pdl_trigger();
    __shared__ float bv[AB / 32];
    __shared__ int bi[AB / 32];
    ti_pdl_sync();
    logits = ti_dependent(logits);
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * ld;
    const int lo = blockIdx.y * per, hi = min(V, lo + per);
    float best = -INFINITY;
    int idx = INT_MAX;
    auto take = [&](float v, int i) { if (v > best || (v == best && i < idx)) { best = v; idx = i; } };
    if ((ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0 && (per & 3) == 0) {
        const int hi4 = lo + ((hi - lo) & ~3);
        for (int i = lo + threadIdx.x * 4; i < hi4; i += AB * 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + i);
            take(v.x, i); take(v.y, i + 1); take(v.z, i + 2); take(v.w, i + 3);
        }
        for (int i = hi4 + threadIdx.x; i < hi; i += AB) take(x[i], i);
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += AB) take(x[i], i);
    }
    auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, best, o);
        const int j = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(w, j, best, idx)) { best = w; idx = j; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < AB / 32 ? bv[lane] : -INFINITY;
        idx = lane < AB / 32 ? bi[lane] : INT_MAX;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, best, o);
            const int j = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(w, j, best, idx)) { best = w; idx = j; }
        }
        if (lane == 0) {
            if (gridDim.y == 1) {
                out[row] = idx == INT_MAX ? 0 : idx;
                return;
            }
            if (idx != INT_MAX) atomicMax(best_word + row, pack_best(best, idx));
            __threadfence();
            if (atomicAdd(tickets + row, 1) == (int)gridDim.y - 1) {
                __threadfence();
                const unsigned long long w = atomicExch(best_word + row, 0ull);
                out[row] = w ? (int)(0xFFFFFFFFu - (unsigned)(w & 0xFFFFFFFFull)) : 0;
                tickets[row] = 0;
            }
        }
    }
}

struct SampleArgs {
    const float* logits; long long ld; int V;
    float temperature; int top_k; float top_p;
    unsigned long long seed; const long long* keys; const int* steps;
    int* out;
};

// top_k in [1, MAXK], top_k < V.  Keeps exactly top_k entries (ties at the k-th value
// go to the lowest indices), then applies top_p on the sorted list.
__global__ void __launch_bounds__(SB) sample_topk_kernel(SampleArgs a) {
    ti_pdl_trigger();
    __shared__ int hist[256];
    __shared__ float cval[MAXK];
    __shared__ int cidx[MAXK];
    __shared__ int scan_i[33];
    __shared__ unsigned s_prefix;
    __shared__ int s_rem, s_count;
    ti_pdl_sync();
    const int t = threadIdx.x, V = a.V, k = a.top_k;
    const float* x = a.logits + (size_t)blockIdx.x * a.ld;
    const float temp = a.temperature;

    // --- the key of the k-th largest value, by radix selection from the top byte down
    unsigned prefix = 0, mask = 0;
    int rem = k;
    for (int pass = 3; pass >= 0; pass--) {
        if (t < 256) hist[t] = 0;
        __syncthreads();
        for (int i = t; i < V; i += SB) {
            const unsigned key = order_key(x[i] / temp);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * pass)) & 255], 1);
        }
        __syncthreads();
        if (t == 0) {
            int above = 0, bin = 255;
            for (; bin > 0; bin--) {
                if (above + hist[bin] >= rem) break;
                above += hist[bin];
            }
            s_prefix = prefix | ((unsigned)bin << (8 * pass));
            s_rem = rem - above;
        }
        __syncthreads();
        prefix = s_prefix;
        rem = s_rem;
        mask |= 0xFFu << (8 * pass);
        __syncthreads();
    }
    const unsigned thr = prefix;   // rem = how many entries equal to thr are kept

    // --- gather: everything above thr, then the `rem` lowest-index entries equal to thr
    if (t == 0) s_count = 0;
    __syncthreads();
    const int chunk = (V + SB - 1) / SB;
    const int lo = min(V, t * chunk), hi = min(V, lo + chunk);
    int ties = 0;
    for (int i = lo; i < hi; i++) {
        const float v = x[i] / temp;
        const unsigned key = order_key(v);
        if (key > thr) {
            const int p = atomicAdd(&s_count, 1);
            if (p < MAXK) { cval[p] = v; cidx[p] = i; }
        } else if (key == thr) {
            ties++;
        }
    }
    int total_ties;
    int rank = block_exclusive_scan<int>(ties, &total_ties, scan_i);
    __syncthreads();
    const int n_gt = s_count;     // < k
    for (int i = lo; i < hi && rank < rem; i++) {
        const float v = x[i] / temp;
        if (order_key(v) == thr) {
            const int p = n_gt + rank;
            if (p < MAXK) { cval[p] = v; cidx[p] = i; }
            rank++;
        }
    }
    __syncthreads();
    const int n = min(k, MAXK);

    // --- sort descending by value, ascending index on ties (bitonic, padded to a power of two)
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    for (int i = n + t; i < n2; i += SB) { cval[i] = -INFINITY; cidx[i] = INT_MAX; }
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = t; i < n2; i += SB) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = (i & size) == 0;
                    const float vi = cval[i], vj = cval[j];
                    const int ii = cidx[i], ij = cidx[j];
                    const bool i_first = vi > vj || (vi == vj && ii < ij);   // i belongs before j
                    if (desc != i_first) { cval[i] = vj; cval[j] = vi; cidx[i] = ij; cidx[j] = ii; }
                }
            }
            __syncthreads();
        }
    }

    // --- softmax over the kept entries, top-p cut, draw
    const float mx = cval[0];
    for (int i = t; i < n; i += SB) cval[i] = expf(cval[i] - mx);
    __syncthreads();
    if (t == 0) {
        float sum = 0.f;
        for (int i = 0; i < n; i++) sum += cval[i];
        float acc = 0.f;
        int kept = n;
        for (int i = 0; i < n; i++) {
            acc += cval[i] / sum;
            if (acc > a.top_p) { kept = i + 1; break; }
        }
        const float u = uniform_from(a.seed, (unsigned long long)a.keys[blockIdx.x],
                                     (unsigned long long)a.steps[blockIdx.x]);
        const float coin = u * acc;
        float run = 0.f;
        int pick = cidx[kept - 1];
        for (int i = 0; i < kept; i++) {
            run += cval[i] / sum;
            if (run > coin) { pick = cidx[i]; break; }
        }
        a.out[blockIdx.x] = pick;
    }
}

// ---------------------------------------------------------------------------
// Any top_k and any top_p, in tiers of MAXK candidates.
//
// The rule is the one of the kernel above (the reference's, src/sampler.cpp:24-68): the kept
// set is the k largest of x = logit / temperature (all of them when top_k is off), p = softmax
// over the kept set, the sorted list is cut after the first entry at which the running sum
// exceeds top_p, and a uniform draw times the sum at the cut picks the first entry whose
// running sum exceeds it.  Entries are ordered by value, larger first, and by index among
// equal values.  The sorted list is never formed as a whole: tier t holds the entries ranked
// t * MAXK ... (t + 1) * MAXK - 1 in that order, found by radix selection of the two ranks that
// bound it (integer counts only, so the result does not depend on the order in which threads
// run), sorted in shared memory and walked by one thread with the running sum carried from tier
// to tier.  A peaked distribution ends in the first tier; a flat one over a large vocabulary
// walks many (a nucleus of 34,000 entries: 34 tiers).  The kept set's sum is formed first, in a
// fixed order (a contiguous run of entries per thread, then a scan over the threads).
// ---------------------------------------------------------------------------
constexpr int MAX_TIERS = 1024;

// Entries at or before a rank in sorted order: key > thr, or key == thr and index <= idx.
struct Bound { unsigned thr; int idx; };

__device__ __forceinline__ bool within(const Bound& b, unsigned key, int i) {
    return key > b.thr || (key == b.thr && i <= b.idx);
}

// The bound of sorted rank `k` (1 <= k <= V): the k entries at or before it are exactly the k
// first of the sorted order.  All threads call it and get the same answer.
__device__ Bound select_rank(const float* x, int V, float temp, int k, int* hist, int* scan_i, unsigned* s_prefix,
                             int* s_rem, int* s_idx) {
    const int t = threadIdx.x;
    unsigned prefix = 0, mask = 0;
    int rem = k, at_thr = 0;
    for (int pass = 3; pass >= 0; pass--) {
        if (t < 256) hist[t] = 0;
        __syncthreads();
        for (int i = t; i < V; i += SB) {
            const unsigned key = order_key(x[i] / temp);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * pass)) & 255], 1);
        }
        __syncthreads();
        if (t == 0) {
            int above = 0, bin = 255;
            for (; bin > 0; bin--) {
                if (above + hist[bin] >= rem) break;
                above += hist[bin];
            }
            *s_prefix = prefix | ((unsigned)bin << (8 * pass));
            s_rem[0] = rem - above;
            s_rem[1] = hist[bin];
        }
        __syncthreads();
        prefix = *s_prefix;
        rem = s_rem[0];
        at_thr = s_rem[1];
        mask |= 0xFFu << (8 * pass);
        __syncthreads();
    }
    Bound b{prefix, INT_MAX};
    if (rem >= at_thr) return b;          // every entry equal to the threshold is inside
    // only the `rem` lowest indices among the equal entries are inside: find the rem-th of them
    const int chunk = (V + SB - 1) / SB;
    const int lo = min(V, t * chunk), hi = min(V, lo + chunk);
    int ties = 0;
    for (int i = lo; i < hi; i++) ties += order_key(x[i] / temp) == prefix ? 1 : 0;
    int total;
    int rank = block_exclusive_scan<int>(ties, &total, scan_i);
    if (rank < rem && rank + ties >= rem) {
        for (int i = lo; i < hi; i++)
            if (order_key(x[i] / temp) == prefix && ++rank == rem) { *s_idx = i; break; }
    }
    __syncthreads();
    b.idx = *s_idx;
    __syncthreads();
    return b;
}

__global__ void __launch_bounds__(SB) sample_tiered_kernel(SampleArgs a, const int* skip) {
    ti_pdl_trigger();
    __shared__ int hist[256];
    __shared__ float cval[MAXK];
    __shared__ int cidx[MAXK];
    __shared__ float tier_end[MAX_TIERS];
    __shared__ int scan_i[33];
    __shared__ float scan_f[33];
    __shared__ float red[33];
    __shared__ unsigned s_prefix;
    __shared__ int s_rem[2], s_idx, s_count;
    __shared__ int s_state[3];            // 0: cut found (1) or not, 1: tier to walk for the pick, 2: entries of the cut tier that are kept
    __shared__ float s_coin;
    ti_pdl_sync();
    if (skip && ti_dependent(skip)[blockIdx.x]) return;        // the kernel before this one has drawn for this row
    const int t = threadIdx.x, V = a.V;
    const float* x = a.logits + (size_t)blockIdx.x * a.ld;
    const float temp = a.temperature;
    const int k_eff = (a.top_k <= 0 || a.top_k >= V) ? V : a.top_k;
    const int chunk = (V + SB - 1) / SB;
    const int lo = min(V, t * chunk), hi = min(V, lo + chunk);

    // --- the maximum, and the kept set's sum of exp(x - max) in a fixed order
    float mx = -INFINITY;
    for (int i = t; i < V; i += SB) mx = fmaxf(mx, x[i] / temp);
    mx = warp_max(mx);
    if ((t & 31) == 0) red[t >> 5] = mx;
    __syncthreads();
    if (t < 32) {
        float m2 = warp_max(red[t]);
        if (t == 0) red[32] = m2;
    }
    __syncthreads();
    mx = red[32];
    Bound all{0u, INT_MAX};
    const Bound kept = k_eff < V ? select_rank(x, V, temp, k_eff, hist, scan_i, &s_prefix, s_rem, &s_idx) : all;
    float part = 0.f;
    for (int i = lo; i < hi; i++) {
        const float v = x[i] / temp;
        if (k_eff == V || within(kept, order_key(v), i)) part += expf(v - mx);
    }
    float sum;
    block_exclusive_scan<float>(part, &sum, scan_f);

    // --- walk the tiers
    const int n_tiers = (k_eff + MAXK - 1) / MAXK;
    const float u = uniform_from(a.seed, (unsigned long long)a.keys[blockIdx.x], (unsigned long long)a.steps[blockIdx.x]);
    if (t == 0) { s_state[0] = 0; s_state[1] = -1; s_state[2] = 0; }
    Bound before = all;                   // rank tier * MAXK; unused for the first tier
    int tier = 0;
    bool picking = false;                 // second visit of an earlier tier, for the pick only
    float acc = 0.f;                      // thread 0: the running sum at the start of the tier
    while (true) {
        const int first = tier * MAXK, m = min(MAXK, k_eff - first);
        const Bound upto = first + m < V ? select_rank(x, V, temp, first + m, hist, scan_i, &s_prefix, s_rem, &s_idx) : all;
        const bool open_end = first + m >= V;
        if (t == 0) s_count = 0;
        __syncthreads();
        for (int i = lo; i < hi; i++) {
            const float v = x[i] / temp;
            const unsigned key = order_key(v);
            if ((open_end || within(upto, key, i)) && (tier == 0 || !within(before, key, i))) {
                const int p = atomicAdd(&s_count, 1);
                if (p < MAXK) { cval[p] = v; cidx[p] = i; }
            }
        }
        __syncthreads();
        const int n = min(s_count, MAXK);      // == m unless the row holds NaNs
        int n2 = 1;
        while (n2 < n) n2 <<= 1;
        for (int i = n + t; i < n2; i += SB) { cval[i] = -INFINITY; cidx[i] = INT_MAX; }
        __syncthreads();
        for (int size = 2; size <= n2; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int i = t; i < n2; i += SB) {
                    const int j = i ^ stride;
                    if (j > i) {
                        const bool desc = (i & size) == 0;
                        const float vi = cval[i], vj = cval[j];
                        const int ii = cidx[i], ij = cidx[j];
                        const bool i_first = vi > vj || (vi == vj && ii < ij);
                        if (desc != i_first) { cval[i] = vj; cval[j] = vi; cidx[i] = ij; cidx[j] = ii; }
                    }
                }
                __syncthreads();
            }
        }
        for (int i = t; i < n; i += SB) cval[i] = expf(cval[i] - mx);
        __syncthreads();
        if (t == 0) {
            if (!picking) {
                // first visit: the running sum, until it passes top_p or the kept set ends
                int cut = -1;
                for (int i = 0; i < n; i++) {
                    acc += cval[i] / sum;
                    if (acc > a.top_p) { cut = i; break; }
                }
                tier_end[tier] = acc;
                if (cut >= 0 || tier == n_tiers - 1) {
                    s_state[0] = 1;
                    s_state[2] = cut >= 0 ? cut + 1 : n;
                    const float coin = u * acc;
                    s_coin = coin;
                    int tp = tier;                       // the first tier whose end passes the coin
                    for (int j = 0; j < tier; j++)
                        if (tier_end[j] > coin) { tp = j; break; }
                    s_state[1] = tp;
                }
            }
        }
        __syncthreads();
        if (s_state[0] && s_state[1] == tier) {
            // the pick lies in the tier that is in shared memory now
            if (t == 0) {
                const int kept_here = picking ? n : s_state[2];
                float run = tier > 0 ? tier_end[tier - 1] : 0.f;
                int pick = kept_here > 0 ? cidx[kept_here - 1] : 0;
                for (int i = 0; i < kept_here; i++) {
                    run += cval[i] / sum;
                    if (run > s_coin) { pick = cidx[i]; break; }
                }
                a.out[blockIdx.x] = pick;
            }
            return;
        }
        if (s_state[0]) {                 // the pick lies in an earlier tier: bring that one back
            picking = true;
            tier = s_state[1];
            before = tier > 0 ? select_rank(x, V, temp, tier * MAXK, hist, scan_i, &s_prefix, s_rem, &s_idx) : all;
        } else {
            before = upto;
            tier++;
        }
        __syncthreads();
    }
}

// whole vocabulary, no top-k, no top-p: first index whose running probability exceeds u
__global__ void __launch_bounds__(SB) sample_full_kernel(SampleArgs a) {
    ti_pdl_trigger();
    __shared__ float red[33];
    __shared__ float scan_f[33];
    __shared__ int s_owner;
    ti_pdl_sync();
    const int t = threadIdx.x, V = a.V;
    const float* x = a.logits + (size_t)blockIdx.x * a.ld;
    const float temp = a.temperature;
    float mx = -INFINITY;
    for (int i = t; i < V; i += SB) mx = fmaxf(mx, x[i] / temp);
    mx = warp_max(mx);
    if ((t & 31) == 0) red[t >> 5] = mx;
    __syncthreads();
    if (t < 32) {
        float m2 = red[t];
        m2 = warp_max(m2);
        if (t == 0) red[32] = m2;
    }
    __syncthreads();
    mx = red[32];
    const int chunk = (V + SB - 1) / SB;
    const int lo = min(V, t * chunk), hi = min(V, lo + chunk);
    float part = 0.f;
    for (int i = lo; i < hi; i++) part += expf(x[i] / temp - mx);
    float total;
    const float off = block_exclusive_scan<float>(part, &total, scan_f);
    const float u = uniform_from(a.seed, (unsigned long long)a.keys[blockIdx.x],
                                 (unsigned long long)a.steps[blockIdx.x]);
    const float target = u * total;
    if (t == 0) s_owner = SB;
    __syncthreads();
    if (hi > lo && off + part > target) atomicMin(&s_owner, t);
    __syncthreads();
    int owner = s_owner;
    if (owner == SB) {   // rounding left the target at the very end: last thread that has entries
        owner = min(SB - 1, (V - 1) / chunk);
    }
    if (t == owner) {
        float acc = off;
        int pick = hi - 1;
        for (int i = lo; i < hi; i++) {
            acc += expf(x[i] / temp - mx);
            if (acc > target) { pick = i; break; }
        }
        a.out[blockIdx.x] = pick;
    }
}

// ---------------------------------------------------------------------------
// The two settings a decode step usually runs with, over many blocks.
//
// One block per row takes 240 us at a vocabulary of 151,936 whatever the setting (a row is 600 KB,
// read four or five times by one SM); a decode step of a 4B-sized model takes 2 to 4 ms.  The two
// usual settings therefore run as two short kernels: the first over (row, chunk of 4,096
// positions) blocks, the second one block per row over what the first left in `scratch`.
//   * top_k up to 1,024 (with or without top_p): an entry is one 64-bit word (value, larger first;
//     index among equal values: the order of the kernels above).  A chunk's block selects its
//     top_k largest words; the second kernel selects the top_k largest of all chunks' candidates
//     (an entry among the top_k of the row is among the top_k of its chunk), sorts them and goes
//     on as sample_topk_kernel does, with the same arithmetic in the same order: the same token.
//   * no top_k, no top_p: a chunk's block leaves the chunk's maximum m and sum of exp(x - m); the
//     second kernel adds the chunks up in order (each scaled to the row's maximum), finds the chunk
//     the draw falls into and walks that chunk.
//   * top_p without top_k: both of the above with 64 candidates per chunk; where the running sum of
//     the row's 64 largest passes top_p (the usual case) the second kernel draws among them and
//     marks the row done; the tiered kernel runs after it and leaves such rows alone.
// ---------------------------------------------------------------------------
constexpr int CHUNK = 4096;       // positions of a row per block of the first kernel
constexpr int NUCLEUS_K = 64;     // candidates within which a nucleus (top_p without top_k) is looked for first
constexpr int CB = 512;           // threads of the first kernels

// An entry as one word: a larger word comes earlier in sorted order (larger value; lower index
// among equal values; -0 counts as +0, as in a float comparison).  0 is no entry.
__device__ __forceinline__ unsigned long long pack_entry(float v, int i) {
    if (v == 0.f) v = 0.f;
    return ((unsigned long long)order_key(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
}
__device__ __forceinline__ float entry_value(unsigned long long w) {
    const unsigned key = (unsigned)(w >> 32);
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key);
}
__device__ __forceinline__ int entry_index(unsigned long long w) { return (int)(0xFFFFFFFFu - (unsigned)(w & 0xFFFFFFFFull)); }

// sorts w[0 .. n2) (n2 a power of two) into descending order; all threads of the block call it
__device__ void sort_descending(unsigned long long* w, int n2) {
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < n2; i += blockDim.x) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = (i & size) == 0;
                    const unsigned long long wi = w[i], wj = w[j];
                    if (desc != (wi > wj)) { w[i] = wj; w[j] = wi; }
                }
            }
            __syncthreads();
        }
    }
}

// The k largest of the block's words (EPT per thread in registers, 0 = none, all others distinct):
// the word of rank k by radix selection, a byte at a time from the top (counts only, so the answer
// does not depend on the order in which threads run), then every word at or above it goes to
// out[0 .. k) in no particular order.  Fewer than k words: all of them, the rest of out is 0.
// hist: 256 ints, s: 3 ints of shared memory.  All threads of the block call it.
template <int EPT>
__device__ void select_largest(const unsigned long long (&w)[EPT], int k, unsigned long long* out, int* hist, int* s) {
    const int t = threadIdx.x;
    unsigned long long prefix = 0, mask = 0;
    int rem = k;
    bool short_of = false;
    for (int pass = 7; pass >= 0; pass--) {
        for (int i = t; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
#pragma unroll
        for (int e = 0; e < EPT; e++)
            if (w[e] != 0ull && (w[e] & mask) == prefix) atomicAdd(&hist[(int)((w[e] >> (8 * pass)) & 255ull)], 1);
        __syncthreads();
        if (t == 0) {
            int above = 0, bin = 255;
            for (; bin > 0; bin--) {
                if (above + hist[bin] >= rem) break;
                above += hist[bin];
            }
            s[0] = bin; s[1] = rem - above;
            s[2] = (above + hist[bin] < rem) ? 1 : (hist[bin] == rem - above ? 2 : 0);      // 1: fewer words than asked for; 2: the bin is taken whole
        }
        __syncthreads();
        prefix |= (unsigned long long)s[0] << (8 * pass);
        rem = s[1];
        const int state = s[2];
        mask |= 255ull << (8 * pass);
        __syncthreads();
        if (state == 1) { short_of = true; break; }
        if (state == 2) break;      // every word that shares the prefix so far is inside: the lower bytes decide nothing
    }
    const unsigned long long thr = short_of ? 1ull : prefix;      // the word of rank k or a lower bound with the same words above it
    if (t == 0) s[0] = 0;
    for (int i = t; i < k; i += blockDim.x) out[i] = 0ull;
    __syncthreads();
#pragma unroll
    for (int e = 0; e < EPT; e++)
        if (w[e] != 0ull && w[e] >= thr) {
            const int p = atomicAdd(&s[0], 1);
            if (p < k) out[p] = w[e];
        }
    __syncthreads();
}

// The same over n words in memory (read once per byte looked at).
__device__ void select_largest_of(const unsigned long long* w, int n, int k, unsigned long long* out, int* hist, int* s) {
    const int t = threadIdx.x;
    unsigned long long prefix = 0, mask = 0;
    int rem = k;
    bool short_of = false;
    for (int pass = 7; pass >= 0; pass--) {
        for (int i = t; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int i = t; i < n; i += blockDim.x) {
            const unsigned long long v = w[i];
            if (v != 0ull && (v & mask) == prefix) atomicAdd(&hist[(int)((v >> (8 * pass)) & 255ull)], 1);
        }
        __syncthreads();
        if (t == 0) {
            int above = 0, bin = 255;
            for (; bin > 0; bin--) {
                if (above + hist[bin] >= rem) break;
                above += hist[bin];
            }
            s[0] = bin; s[1] = rem - above;
            s[2] = (above + hist[bin] < rem) ? 1 : (hist[bin] == rem - above ? 2 : 0);
        }
        __syncthreads();
        prefix |= (unsigned long long)s[0] << (8 * pass);
        rem = s[1];
        const int state = s[2];
        mask |= 255ull << (8 * pass);
        __syncthreads();
        if (state == 1) { short_of = true; break; }
        if (state == 2) break;
    }
    const unsigned long long thr = short_of ? 1ull : prefix;
    if (t == 0) s[0] = 0;
    for (int i = t; i < k; i += blockDim.x) out[i] = 0ull;
    __syncthreads();
    for (int i = t; i < n; i += blockDim.x) {
        const unsigned long long v = w[i];
        if (v != 0ull && v >= thr) {
            const int p = atomicAdd(&s[0], 1);
            if (p < k) out[p] = v;
        }
    }
    __syncthreads();
}

constexpr int K1B = 256;      // threads of the chunk kernel: 16 entries each

// the block's sum of v in a fixed order (threads in order within a warp's tree, warps in order)
__device__ float block_sum_ordered(float v, float* sm /* 33 entries */) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) s += sm[i];
        sm[32] = s;
    }
    __syncthreads();
    return sm[32];
}

// The block's chunk: its k largest entries to cand[row][chunk][0 .. k), and, with `stats`, the
// chunk's maximum m and sum of exp(x - m) (as softmax_chunk_kernel leaves them).
__global__ void __launch_bounds__(K1B) topk_chunk_kernel(SampleArgs a, int k, int chunks, unsigned long long* cand, float* stats) {
    ti_pdl_trigger();
    __shared__ int hist[256];
    __shared__ int sh[3];
    __shared__ float red[33];
    __shared__ unsigned long long kept[MAXK];
    ti_pdl_sync();
    const int row = blockIdx.x, c = blockIdx.y, lo = c * CHUNK, t = threadIdx.x;
    const int n = min(CHUNK, a.V - lo);
    const float* x = a.logits + (size_t)row * a.ld + lo;
    unsigned long long w[CHUNK / K1B];
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < CHUNK / K1B; e++) {
        const int i = t + e * K1B;
        const float v = i < n ? x[i] / a.temperature : -INFINITY;
        w[e] = i < n ? pack_entry(v, lo + i) : 0ull;
        mx = fmaxf(mx, v);
    }
    if (stats) {
        mx = warp_max(mx);
        if ((t & 31) == 0) red[t >> 5] = mx;
        __syncthreads();
        if (t < 32) {
            float m2 = warp_max(t < K1B / 32 ? red[t] : -INFINITY);
            if (t == 0) red[32] = m2;
        }
        __syncthreads();
        mx = red[32];
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < CHUNK / K1B; e++) part += (w[e] != 0ull && mx > -INFINITY) ? expf(entry_value(w[e]) - mx) : 0.f;
        const float sum = block_sum_ordered(part, red);
        if (t == 0) {
            stats[((size_t)row * chunks + c) * 2] = mx;
            stats[((size_t)row * chunks + c) * 2 + 1] = sum;
        }
    }
    select_largest<CHUNK / K1B>(w, k, kept, hist, sh);
    unsigned long long* out = cand + ((size_t)row * chunks + c) * k;
    for (int i = t; i < k; i += K1B) out[i] = kept[i];
}

// The row's k largest among the chunks' candidates, sorted, in kept[0 .. k) (the rest of kept up to
// the next power of two is 0).  All threads call it.
__device__ int merge_candidates(const unsigned long long* cand, int n_cand, int k, unsigned long long* kept, int* hist, int* sh) {
    int n2 = 1;
    while (n2 < k) n2 <<= 1;
    for (int i = threadIdx.x; i < n2; i += blockDim.x) kept[i] = 0ull;
    __syncthreads();
    select_largest_of(cand, n_cand, k, kept, hist, sh);
    sort_descending(kept, n2);
    return n2;
}

__global__ void __launch_bounds__(SB) topk_merge_kernel(SampleArgs a, int chunks, const unsigned long long* cand) {
    ti_pdl_trigger();
    __shared__ int hist[256];
    __shared__ int sh[3];
    __shared__ unsigned long long kept[MAXK];
    __shared__ float cval[MAXK];
    ti_pdl_sync();
    cand = ti_dependent(cand);
    const int t = threadIdx.x, row = blockIdx.x, k = a.top_k;
    merge_candidates(cand + (size_t)row * chunks * k, chunks * k, k, kept, hist, sh);
    // --- softmax over the kept entries, top-p cut, draw: as in sample_topk_kernel
    const int n = k;                            // top_k < V: there are that many entries
    const float mx = entry_value(kept[0]);
    for (int i = t; i < n; i += SB) cval[i] = expf(entry_value(kept[i]) - mx);
    __syncthreads();
    if (t == 0) {
        float sum = 0.f;
        for (int i = 0; i < n; i++) sum += cval[i];
        float acc = 0.f;
        int keep = n;
        for (int i = 0; i < n; i++) {
            acc += cval[i] / sum;
            if (acc > a.top_p) { keep = i + 1; break; }
        }
        const float u = uniform_from(a.seed, (unsigned long long)a.keys[row], (unsigned long long)a.steps[row]);
        const float coin = u * acc;
        float run = 0.f;
        int pick = entry_index(kept[keep - 1]);
        for (int i = 0; i < keep; i++) {
            run += cval[i] / sum;
            if (run > coin) { pick = entry_index(kept[i]); break; }
        }
        a.out[row] = pick;
    }
}

// top_p without top_k: the row's NUCLEUS_K largest entries and the whole row's sum of exponentials.
// Where the running sum of those entries' probabilities passes top_p, the nucleus lies within
// them: the draw is made here (sample_tiered_kernel's rule: p = exp(x - max) / the row's sum, in
// sorted order; the list ends with the first entry at which the running sum exceeds top_p; the
// uniform number times the sum at that point picks the first entry whose running sum exceeds it)
// and done[row] is set; else done[row] = 0 and the tiered kernel, which runs next, does the row.
__global__ void __launch_bounds__(SB) nucleus_merge_kernel(SampleArgs a, int chunks, const unsigned long long* cand, const float* stats,
                                                           int* done) {
    ti_pdl_trigger();
    __shared__ int hist[256];
    __shared__ int sh[3];
    __shared__ unsigned long long kept[NUCLEUS_K];
    ti_pdl_sync();
    cand = ti_dependent(cand); stats = ti_dependent(stats);
    const int t = threadIdx.x, row = blockIdx.x;
    const int k = min(NUCLEUS_K, a.V);
    merge_candidates(cand + (size_t)row * chunks * NUCLEUS_K, chunks * NUCLEUS_K, k, kept, hist, sh);
    if (t == 0) {
        const float* st = stats + (size_t)row * chunks * 2;
        float mx = -INFINITY;
        for (int c = 0; c < chunks; c++) mx = fmaxf(mx, st[2 * c]);
        float sum = 0.f;
        for (int c = 0; c < chunks; c++) sum += st[2 * c] > -INFINITY ? st[2 * c + 1] * expf(st[2 * c] - mx) : 0.f;
        float acc = 0.f;
        int keep = 0;
        for (int i = 0; i < k && kept[i] != 0ull; i++) {
            acc += expf(entry_value(kept[i]) - mx) / sum;
            if (acc > a.top_p) { keep = i + 1; break; }
        }
        if (keep == 0 && k == a.V) keep = k;            // a vocabulary this small is in `kept` whole
        if (keep > 0) {
            const float u = uniform_from(a.seed, (unsigned long long)a.keys[row], (unsigned long long)a.steps[row]);
            const float coin = u * acc;
            float run = 0.f;
            int pick = entry_index(kept[keep - 1]);
            for (int i = 0; i < keep; i++) {
                run += expf(entry_value(kept[i]) - mx) / sum;
                if (run > coin) { pick = entry_index(kept[i]); break; }
            }
            a.out[row] = pick;
        }
        done[row] = keep > 0 ? 1 : 0;
    }
}

__global__ void __launch_bounds__(CB) softmax_chunk_kernel(SampleArgs a, int chunks, float* stats) {
    ti_pdl_trigger();
    __shared__ float red[33];
    ti_pdl_sync();
    const int row = blockIdx.x, c = blockIdx.y, lo = c * CHUNK, t = threadIdx.x;
    const int n = min(CHUNK, a.V - lo);
    const float* x = a.logits + (size_t)row * a.ld + lo;
    float v[CHUNK / CB];
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < CHUNK / CB; e++) {
        const int i = t + e * CB;
        v[e] = i < n ? x[i] / a.temperature : -INFINITY;
        mx = fmaxf(mx, v[e]);
    }
    mx = warp_max(mx);
    if ((t & 31) == 0) red[t >> 5] = mx;
    __syncthreads();
    if (t < 32) {
        float m2 = warp_max(t < CB / 32 ? red[t] : -INFINITY);
        if (t == 0) red[32] = m2;
    }
    __syncthreads();
    mx = red[32];
    float part = 0.f;
#pragma unroll
    for (int e = 0; e < CHUNK / CB; e++) part += (t + e * CB < n && mx > -INFINITY) ? expf(v[e] - mx) : 0.f;
    const float sum = block_sum_ordered(part, red);
    if (t == 0) {
        stats[((size_t)row * chunks + c) * 2] = mx;
        stats[((size_t)row * chunks + c) * 2 + 1] = sum;
    }
}

__global__ void __launch_bounds__(CB) sample_full_merge_kernel(SampleArgs a, int chunks, const float* stats) {
    ti_pdl_trigger();
    __shared__ float scan_f[33];
    __shared__ int s_chunk, s_pick;
    __shared__ float s_mx, s_before, s_target;
    ti_pdl_sync();
    stats = ti_dependent(stats);
    const int row = blockIdx.x, t = threadIdx.x;
    const float* st = stats + (size_t)row * chunks * 2;
    if (t == 0) {
        float mx = -INFINITY;
        for (int c = 0; c < chunks; c++) mx = fmaxf(mx, st[2 * c]);
        // a chunk's sum, scaled from its own maximum to the row's
        auto weight = [&](int c) { return st[2 * c] > -INFINITY ? st[2 * c + 1] * expf(st[2 * c] - mx) : 0.f; };
        float total = 0.f;
        for (int c = 0; c < chunks; c++) total += weight(c);
        const float u = uniform_from(a.seed, (unsigned long long)a.keys[row], (unsigned long long)a.steps[row]);
        const float target = u * total;
        // the first chunk at whose end the running sum exceeds the target (rounding may leave none: the last)
        float run = 0.f;
        int pick = -1;
        for (int c = 0; c < chunks; c++) {
            const float w = weight(c);
            if (run + w > target) { pick = c; break; }
            run += w;
        }
        if (pick < 0) { pick = chunks - 1; run -= weight(pick); }
        s_chunk = pick; s_mx = mx; s_before = run; s_target = target;
        s_pick = INT_MAX;
    }
    __syncthreads();
    const int lo = s_chunk * CHUNK;
    const int n = min(CHUNK, a.V - lo);
    const float* x = a.logits + (size_t)row * a.ld + lo;
    const float mx = s_mx, target = s_target;
    float base = s_before;
    // walk the chunk in runs of CB positions: the first position whose running sum exceeds the target
    for (int i0 = 0; i0 < n; i0 += CB) {
        const int i = i0 + t;
        const float e = i < n ? expf(x[i] / a.temperature - mx) : 0.f;
        float total;
        const float off = block_exclusive_scan<float>(e, &total, scan_f);
        if (i < n && base + off + e > target) atomicMin(&s_pick, i);
        __syncthreads();
        if (s_pick != INT_MAX) break;
        base += total;
    }
    if (t == 0) a.out[row] = lo + (s_pick != INT_MAX ? s_pick : n - 1);     // rounding left the target at the very end: the last position
}

}  // namespace

// best_word[R] (64-bit) and tickets[R] are scratch that is zero before the first call and
// left zero; calls that share them must be on one stream.  They may be null: one block per
// row then.
extern "C" int ti_argmax(const float* logits, long long ld, int R, int V, int sms, unsigned long long* best_word,
                         int* tickets, int* out, cudaStream_t stream) {
    if (R == 0) return 0;
    TI_REQUIRE(R > 0 && V > 0 && ld >= V, "argmax: bad sizes R=%d V=%d ld=%lld", R, V, ld);
    int chunks = 1;
    if (best_word && tickets) {
        chunks = (2 * (sms > 0 ? sms : 1)) / R;                      // about two blocks per SM
        const int most = (V + 4 * AB - 1) / (4 * AB);                // at least one vector per thread
        if (chunks > most) chunks = most;
        if (chunks > 64) chunks = 64;
        if (chunks < 1) chunks = 1;
    }
    int per = ((V + chunks - 1) / chunks + 3) & ~3;
    chunks = (V + per - 1) / per;
    TI_REQUIRE(chunks <= 65535, "argmax: too many chunks");
    TI_CUDA(ti_launch(argmax_kernel, dim3(R, chunks), dim3(AB), 0, stream, logits, ld, V, per, best_word, tickets, out));
    TI_CHECK_LAUNCH("argmax");
    return 0;
}

// keys[R] (int64) and steps[R] (int32) on the device name each row's sequence and how many
// tokens it has drawn so far.
// Bytes of scratch with which ti_sample runs this setting as two short kernels over many blocks
// (0: it has only the one-block-per-row form for it).
extern "C" long long ti_sample_scratch_bytes(int R, int V, int top_k, float top_p) {
    if (R <= 0 || V <= 0) return 0;
    const long long chunks = (V + CHUNK - 1) / CHUNK;
    const bool k_off = top_k <= 0 || top_k >= V;
    const long long stats = (long long)R * chunks * 2 * (long long)sizeof(float);
    if (k_off && top_p >= 1.0f) return stats;
    if (!k_off && top_k <= MAXK) return (long long)R * chunks * top_k * (long long)sizeof(unsigned long long);
    if (k_off) return (long long)R * chunks * NUCLEUS_K * (long long)sizeof(unsigned long long) + stats + (long long)R * (long long)sizeof(int);
    return 0;
}

// `scratch`: ti_sample_scratch_bytes(...) bytes, 8-byte aligned, or null (one block per row then).
extern "C" int ti_sample(const float* logits, long long ld, int R, int V, float temperature, int top_k,
                         float top_p, unsigned long long seed, const long long* keys, const int* steps,
                         int* out, void* scratch, cudaStream_t stream) {
    if (R == 0) return 0;
    TI_REQUIRE(R > 0 && V > 0 && ld >= V, "sample: bad sizes R=%d V=%d ld=%lld", R, V, ld);
    TI_REQUIRE(temperature > 0.f, "sample: temperature %g must be positive (zero is the argmax rule)", temperature);
    TI_REQUIRE(top_p > 0.f, "sample: top_p %g must be positive", top_p);
    SampleArgs a;
    a.logits = logits; a.ld = ld; a.V = V; a.temperature = temperature; a.top_k = top_k;
    a.top_p = top_p; a.seed = seed; a.keys = keys; a.steps = steps; a.out = out;
    const bool k_off = top_k <= 0 || top_k >= V;
    const int chunks = (V + CHUNK - 1) / CHUNK;
    if (scratch && ti_sample_scratch_bytes(R, V, top_k, top_p) > 0) {
        TI_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 7) == 0 && chunks <= 65535, "sample: bad scratch or too many chunks");
        if (k_off && top_p >= 1.0f) {
            TI_CUDA(ti_launch(softmax_chunk_kernel, dim3(R, chunks), dim3(CB), 0, stream, a, chunks, (float*)scratch));
            TI_CUDA(ti_launch(sample_full_merge_kernel, dim3(R), dim3(CB), 0, stream, a, chunks, (const float*)scratch));
        } else if (!k_off) {
            TI_CUDA(ti_launch(topk_chunk_kernel, dim3(R, chunks), dim3(K1B), 0, stream, a, top_k, chunks, (unsigned long long*)scratch, (float*)nullptr));
            TI_CUDA(ti_launch(topk_merge_kernel, dim3(R), dim3(SB), 0, stream, a, chunks, (const unsigned long long*)scratch));
        } else {
            unsigned long long* cand = (unsigned long long*)scratch;
            float* stats = (float*)(cand + (size_t)R * chunks * NUCLEUS_K);
            int* done = (int*)(stats + (size_t)R * chunks * 2);
            TI_CUDA(ti_launch(topk_chunk_kernel, dim3(R, chunks), dim3(K1B), 0, stream, a, NUCLEUS_K, chunks, cand, stats));
            TI_CUDA(ti_launch(nucleus_merge_kernel, dim3(R), dim3(SB), 0, stream, a, chunks, (const unsigned long long*)cand, (const float*)stats, done));
            TI_CUDA(ti_launch(sample_tiered_kernel, dim3(R), dim3(SB), 0, stream, a, (const int*)done));
        }
        TI_CHECK_LAUNCH("sample");
        return 0;
    }
    if (k_off && top_p >= 1.0f) {
        TI_CUDA(ti_launch(sample_full_kernel, dim3(R), dim3(SB), 0, stream, a));
    } else if (!k_off && top_k <= MAXK) {
        TI_CUDA(ti_launch(sample_topk_kernel, dim3(R), dim3(SB), 0, stream, a));
    } else {
        // top_p over the whole vocabulary, or more candidates than one sort holds: tier by tier
        const long long kept = k_off ? V : top_k;
        TI_REQUIRE(kept <= (long long)MAXK * MAX_TIERS, "sample: %lld candidates exceed the %d this kernel walks", kept,
                   MAXK * MAX_TIERS);
        TI_CUDA(ti_launch(sample_tiered_kernel, dim3(R), dim3(SB), 0, stream, a, (const int*)nullptr));
    }
    TI_CHECK_LAUNCH("sample");
    return 0;
}

extern "C" float ti_uniform_from(unsigned long long seed, unsigned long long key, unsigned long long step) {
    return uniform_from(seed, key, step);
}

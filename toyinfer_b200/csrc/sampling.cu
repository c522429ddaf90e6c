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

__global__ void __launch_bounds__(SB) sample_tiered_kernel(SampleArgs a) {
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
extern "C" int ti_sample(const float* logits, long long ld, int R, int V, float temperature, int top_k,
                         float top_p, unsigned long long seed, const long long* keys, const int* steps,
                         int* out, cudaStream_t stream) {
    if (R == 0) return 0;
    TI_REQUIRE(R > 0 && V > 0 && ld >= V, "sample: bad sizes R=%d V=%d ld=%lld", R, V, ld);
    TI_REQUIRE(temperature > 0.f, "sample: temperature %g must be positive (zero is the argmax rule)", temperature);
    TI_REQUIRE(top_p > 0.f, "sample: top_p %g must be positive", top_p);
    SampleArgs a;
    a.logits = logits; a.ld = ld; a.V = V; a.temperature = temperature; a.top_k = top_k;
    a.top_p = top_p; a.seed = seed; a.keys = keys; a.steps = steps; a.out = out;
    const bool k_off = top_k <= 0 || top_k >= V;
    if (k_off && top_p >= 1.0f) {
        TI_CUDA(ti_launch(sample_full_kernel, dim3(R), dim3(SB), 0, stream, a));
    } else if (!k_off && top_k <= MAXK) {
        TI_CUDA(ti_launch(sample_topk_kernel, dim3(R), dim3(SB), 0, stream, a));
    } else {
        // top_p over the whole vocabulary, or more candidates than one sort holds: tier by tier
        const long long kept = k_off ? V : top_k;
        TI_REQUIRE(kept <= (long long)MAXK * MAX_TIERS, "sample: %lld candidates exceed the %d this kernel walks", kept,
                   MAXK * MAX_TIERS);
        TI_CUDA(ti_launch(sample_tiered_kernel, dim3(R), dim3(SB), 0, stream, a));
    }
    TI_CHECK_LAUNCH("sample");
    return 0;
}

extern "C" float ti_uniform_from(unsigned long long seed, unsigned long long key, unsigned long long step) {
    return uniform_from(seed, key, step);
}

// Shared by the decode attention kernels: the argument block and the kernel that merges
// the partial results of the splits along the keys.
#pragma once

#include "common.cuh"

namespace tiattn {

struct DecodeArgs {
    const void* q; long long q_stride;        // [B, heads, hd]
    const void* k_pages; const void* v_pages; // [pages, kv_heads, page, hd]
    const int* page_table; int table_width; int page_size; int ring_rows; int n_pages;
    const int* seq_slot; const int* seq_len;
    int n_heads, n_kv_heads, hd, window, n_splits;
    float scale;
    void* out; long long o_stride;            // [B, heads, hd]
    float* part_o; float* part_ml;            // [B, heads, splits, hd], [B, heads, splits, 2]
};

// One block per (sequence, head); threads over the head's elements.  A split that saw no
// key has maximum -inf and contributes nothing.  The splits' weights are worked out once per
// block from shared memory; the sums then run over independent loads, four splits at a time.
template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           T* __restrict__ out, long long o_stride, int n_heads, int hd,
                                           int n_splits) {
    ti_pdl_trigger();
    ti_pdl_sync();
    part_o = ti_dependent(part_o); part_ml = ti_dependent(part_ml);
    __shared__ float w_s[128];       // weight of each split (up to 128 at a time)
    const int b = blockIdx.x, h = blockIdx.y;
    const size_t base = ((size_t)b * n_heads + h) * n_splits;
    // pass over the (maximum, sum) pairs: every thread reads them all (they are few and cached)
    float m = -INFINITY;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, part_ml[(base + s) * 2]);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};         // up to 4 elements per thread (hd <= 4 * blockDim)
    float l = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 128) {
        const int cnt = min(128, n_splits - s0);
        __syncthreads();
        for (int s = threadIdx.x; s < cnt; s += blockDim.x) {
            const float ms = part_ml[(base + s0 + s) * 2];
            w_s[s] = ms > -INFINITY ? expf(ms - m) : 0.f;
        }
        __syncthreads();
        for (int s = 0; s < cnt; s++) {
            const float w = w_s[s], ls = part_ml[(base + s0 + s) * 2 + 1];
            l += w > 0.f ? ls * w : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int d = threadIdx.x + e * blockDim.x;
            if (d < hd) {
                float o = acc[e];
                int s = 0;
                for (; s + 4 <= cnt; s += 4) {
                    const float v0 = part_o[(base + s0 + s) * hd + d], v1 = part_o[(base + s0 + s + 1) * hd + d];
                    const float v2 = part_o[(base + s0 + s + 2) * hd + d], v3 = part_o[(base + s0 + s + 3) * hd + d];
                    const float w0 = w_s[s], w1 = w_s[s + 1], w2 = w_s[s + 2], w3 = w_s[s + 3];
                    // an empty split's numbers were never written: they are dropped, not multiplied by 0
                    o = fmaf(w0 > 0.f ? v0 : 0.f, w0, o); o = fmaf(w1 > 0.f ? v1 : 0.f, w1, o);
                    o = fmaf(w2 > 0.f ? v2 : 0.f, w2, o); o = fmaf(w3 > 0.f ? v3 : 0.f, w3, o);
                }
                for (; s < cnt; s++) {
                    const float w = w_s[s], v = part_o[(base + s0 + s) * hd + d];
                    o = fmaf(w > 0.f ? v : 0.f, w, o);
                }
                acc[e] = o;
            }
        }
    }
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int d = threadIdx.x + e * blockDim.x;
        if (d < hd) out[(size_t)b * o_stride + (size_t)h * hd + d] = from_f32<T>(l > 0.f ? acc[e] / l : 0.f);
    }
}

}  // namespace tiattn

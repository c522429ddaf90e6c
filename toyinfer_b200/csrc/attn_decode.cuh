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
// key has maximum -inf and contributes nothing.
template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           T* __restrict__ out, long long o_stride, int n_heads, int hd,
                                           int n_splits) {
    ti_pdl_trigger();
    ti_pdl_sync();
    const int b = blockIdx.x, h = blockIdx.y;
    const size_t base = ((size_t)b * n_heads + h) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, part_ml[(base + s) * 2]);
    float l = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = part_ml[(base + s) * 2];
        if (ms > -INFINITY) l += part_ml[(base + s) * 2 + 1] * expf(ms - m);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < n_splits; s++) {
            const float ms = part_ml[(base + s) * 2];
            if (ms > -INFINITY) o = fmaf(part_o[(base + s) * hd + d], expf(ms - m), o);
        }
        out[(size_t)b * o_stride + (size_t)h * hd + d] = from_f32<T>(l > 0.f ? o / l : 0.f);
    }
}

}  // namespace tiattn

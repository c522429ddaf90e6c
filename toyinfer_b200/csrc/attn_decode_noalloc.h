// ti_attn_decode_noalloc: split decode attention for callers that must not allocate.
//
// This entry point has no counterpart in wiketool/ToyInfer; it exists for users of this
// library whose code cannot call cudaMalloc at the point where it needs attention over the
// cache: code that runs between a framework's memory-pool checkpoints, real-time loops
// that forbid calls which may take a device-wide lock or synchronise, plugins that are
// handed a fixed memory budget by their host.  The library's usual entry point
// (ti_attn_decode_simt) takes two float32 scratch buffers for the partial results of the
// splits along the keys; this one keeps that scratch inside the library instead, in an
// array of fixed size in device memory (TI_NOALLOC_SCRATCH_FLOATS floats, 4 MiB, held by
// every GPU that loads the library until the process exits).
//
// Same arguments and result as ti_attn_decode_simt, minus the two scratch pointers.
//   * n_seq * n_heads * n_splits * (head_dim + 2) must not exceed
//     TI_NOALLOC_SCRATCH_FLOATS; a larger request is refused with a message
//     (ti_last_error) and nothing is launched.  With n_splits == 1 no scratch is used and
//     any size is taken.
//   * The first call on a device looks up the array's device address (no allocation, but a
//     runtime call that is not allowed while a stream is being captured): make that first
//     call before any capture begins.
//   * All calls share the one array and it keeps what the last call left there.  Nothing in
//     it has to be zero at the start: every split writes its whole partial result, also a
//     split that saw no key, before the merge reads it.  Two calls that overlap on the GPU
//     (different streams, or the same call from two host threads) race on it: run them one
//     after another.
//   * It calls no cudaMalloc, cudaFree or other allocating routine, here or in what it calls.
#pragma once

#include <cuda_runtime.h>

#define TI_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int ti_attn_decode_noalloc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                           const int* page_table, int table_width, int page_size, int ring_rows,
                           int n_pages, const int* seq_slot, const int* seq_len, int n_seq,
                           int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                           int n_splits, void* out, long long o_stride, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

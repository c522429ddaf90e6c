// C entry points around wiketool/ToyInfer's own kernel wrappers (include/kernel_warpper.h), so
// that a measurement can call them from Python.  The reference's kernels are compiled unchanged:
// this file includes its src/kernel.cu (which includes decode.cu and prefill.cu) and adds nothing
// to them.  Template arguments are the ones the reference's engine uses: 256 threads
// (include/config.h:6), sequence tiles of 32 (include/config.h:7), flash attention <32, 4, 128>
// (src/transformer.cpp:26-38).
#include "kernel.cu"

using toyinfer::bf16;

extern "C" {

// y[M] = W[M, N] x[N], bfloat16 out (src/decode.cu:202-247)
void ref_gemv(const void* W, const void* x, void* y, unsigned M, unsigned N, void* stream) {
    toyinfer::gemv_proj_bf16<256>((const bf16*)W, (const bf16*)x, (bf16*)y, M, N, (cudaStream_t)stream);
}

// the same with float32 out: the head (src/decode.cu:251-298)
void ref_gemv_f32(const void* W, const void* x, float* y, unsigned M, unsigned N, void* stream) {
    toyinfer::gemv_proj_bf162float<256>((const bf16*)W, (const bf16*)x, y, M, N, (cudaStream_t)stream);
}

// y[T, M] = x[T, N] W[M, N]^T, one block per output element (src/prefill.cu:124-175)
void ref_batch_gemv(const void* W, const void* x, void* y, unsigned T, unsigned M, unsigned N, void* stream) {
    toyinfer::batch_gemv_proj_bf16<256>((const bf16*)W, (const bf16*)x, (bf16*)y, T, M, N, (cudaStream_t)stream);
}

// causal GQA attention over a whole prompt (src/prefill.cu:224-393)
void ref_flash_attention(const void* Q, const void* K, const void* V, void* O, unsigned n_q_heads, unsigned n_kv_heads,
                         unsigned head_dim, unsigned seq_len, void* stream) {
    toyinfer::flash_attention_v1_bf16<32, 4, 128>((const bf16*)Q, (const bf16*)K, (const bf16*)V, (bf16*)O, n_q_heads,
                                                  n_kv_heads, head_dim, seq_len, (cudaStream_t)stream);
}

// one token's attention over cache rows 0..pos: two memsets and four kernels (src/decode.cu:703-744)
void ref_attention_decode(const void* Q, const void* Ks, const void* Vs, float* score, float* o_buffer, void* O,
                          unsigned n_q_heads, unsigned n_kv_heads, unsigned head_dim, unsigned pos, unsigned max_seq_len,
                          void* stream) {
    toyinfer::attention_bf16<256, 32>((const bf16*)Q, (const bf16*)Ks, (const bf16*)Vs, score, o_buffer, (bf16*)O, n_q_heads,
                                      n_kv_heads, head_dim, pos, max_seq_len, (cudaStream_t)stream);
}

}  // extern "C"

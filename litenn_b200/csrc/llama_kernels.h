// Host-callable launchers of the decoder glue kernels (internal to the library).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmm {

cudaError_t ll_rope_tables(int max_seq, int rope_dim, double theta, float* rope_cos, float* rope_sin, cudaStream_t st);
cudaError_t ll_embed_rows(int fmt, const uint8_t* raw, const int* tokens, int n_rows, int d, float* h, cudaStream_t st);
cudaError_t ll_resid_rmsnorm_pack(const float* h_in, const float* add, const float* w, float eps, int d,
                                  uint8_t* packed, float* h_out, cudaStream_t st);
cudaError_t ll_rope_kv(float* qkv, const int* pos, int pos_add, int rows, int n_heads, int n_kv, int hd, int rope_dim,
                       const float* rope_cos, const float* rope_sin, int max_seq, __half* cache_k, __half* cache_v,
                       cudaStream_t st);
cudaError_t ll_attn_fused(const float* qkv, const int* pos, int n_heads, int n_kv, int hd, int rope_dim,
                          const float* rope_cos, const float* rope_sin, int max_seq, __half* cache_k, __half* cache_v,
                          uint8_t* packed, cudaStream_t st);
cudaError_t ll_silu_mul_pack(const float* gu, int ffn, uint8_t* packed, cudaStream_t st);
cudaError_t ll_argmax(const float* logits, int n, int index_offset, int ctas, int* best_pair, cudaStream_t st);
cudaError_t ll_commit_token(const int* pairs, int ranks, int* token, int* pos, int* out_tokens, int* out_count,
                            cudaStream_t st);
cudaError_t ll_resid_rmsnorm_rows(float* h, const float* add, const float* w, float eps, int d, int64_t m,
                                  __nv_bfloat16* xn, cudaStream_t st);
cudaError_t ll_attn_prefill(const float* qkv, int m, int pos0, int n_heads, int n_kv, int hd, int max_seq,
                            const __half* cache_k, const __half* cache_v, __nv_bfloat16* ctx, cudaStream_t st);
cudaError_t ll_silu_mul_rows(const float* gu, int64_t m, int ffn, __nv_bfloat16* act, cudaStream_t st);
cudaError_t ll_add_rows(float* h, const float* add, int64_t total, cudaStream_t st);

}  // namespace qmm

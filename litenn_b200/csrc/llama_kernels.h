// Host-callable launchers of the decoder glue kernels (internal to the library).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmm {

cudaError_t ll_rope_tables(int max_seq, int rope_dim, double theta, float* rope_cos, float* rope_sin, cudaStream_t st);
cudaError_t ll_embed_rows(int fmt, const uint8_t* raw, const int* tokens, int n_rows, int d, float* h, cudaStream_t st);
// Receiving side of the tensor-parallel sum that PeerScatter (qmm_common.cuh) feeds; tp_size <= 1 = off.
struct PeerGather {
    const uint2* recv;  // [tp_size][d] packets {value bits, exchange number} (own slot unused)
    int tp_rank, tp_size;
    const int* pos;     // exchange number = *pos * sites + site + 1
    int sites, site;
    int* status;        // set to 5 when a packet did not come within the wait limit
    unsigned int spin_limit;  // polls of one packet before giving up
};
// Exchange of the ranks' arg-max winners inside the commit kernel; tp_size <= 1 = off.
struct ArgmaxExchange {
    const uint2* recv;  // [tp_size][2] packets {value bits, number} {index, number} (own slot unused)
    uint2* peer[8];     // the same buffer of every rank, mapped here (own entry unused)
    int tp_rank, tp_size;
    int* status;        // set to 6 when a peer's candidate did not come within the wait limit
    unsigned int spin_limit;
};

// Decode, first kernel of a token: h = embedding row of *token; packed = pack(h * w); ss_out = sums of
// squares per 32 elements (the consumer matvec applies 1/rms).
cudaError_t ll_embed_pack(int fmt, const uint8_t* raw, const int* token, int d, const float* w, float* h,
                          uint8_t* packed, double* ss_out, cudaStream_t st);
// h_out = h_in + add (+ the peers' addends when pg.tp_size > 1); packed = pack(h_out * w); ss_out as above.
cudaError_t ll_resid_pack(const float* h_in, const float* add, const float* w, int d, float* h_out, uint8_t* packed,
                          double* ss_out, const PeerGather& pg, cudaStream_t st);
cudaError_t ll_rope_kv(float* qkv, const int* pos, int pos_add, int rows, int n_heads, int n_kv, int hd, int rope_dim,
                       const float* rope_cos, const float* rope_sin, int max_seq, __half* cache_k, __half* cache_v,
                       cudaStream_t st);
// Batched decode attention (grid.y = sequence): every sequence has its own qkv row, position and cache.
// All zero = one sequence whose context is packed for the attn_output matvec.
struct AttnBatch {
    int qkv_stride;        // floats between the sequences' qkv rows
    int64_t cache_stride;  // halves between the sequences' caches of one block
    float* ctx;            // not null: the context is stored as fp32 rows [batch][ctx_stride] instead of packed
    int ctx_stride;
};
// RoPE of q and the new key, KV append, attention over the cache, for `batch` sequences (pos[batch]).
cudaError_t ll_attn_fused(const float* qkv, const int* pos, int n_heads, int n_kv, int hd, int rope_dim,
                          const float* rope_cos, const float* rope_sin, int max_seq, __half* cache_k, __half* cache_v,
                          uint8_t* packed, int batch, const AttnBatch& ab, cudaStream_t st);
// `rows` rows of logits `row_stride` apart; candidates of row r at best_pair[r * 2 * ctas ..].
cudaError_t ll_argmax(const float* logits, int n, int index_offset, int ctas, int* best_pair, int rows,
                      int64_t row_stride, cudaStream_t st);
// Batched decode: winner per row over pairs[ranks][batch][2 * per_rank]; tokens[row], pos[row]++,
// out_tokens[*out_steps][row], (*out_steps)++.
cudaError_t ll_commit_batch(const int* pairs, int per_rank, int ranks, int batch, int* tokens, int* pos, int* out_tokens,
                            int* out_steps, cudaStream_t st);
// Where the commit kernel also leaves {token, model status word, library status word} for the host
// (mapped pinned memory; host == null switches it off).
struct TokenReport {
    int* host;
    const int* model_status;
    const int* library_status;
};
cudaError_t ll_commit_token(const int* pairs, int n_local, const ArgmaxExchange& ax, int* token, int* pos,
                            int* out_tokens, int* out_count, const TokenReport& report, cudaStream_t st);
cudaError_t ll_resid_rmsnorm_rows(float* h, const float* add, const float* w, float eps, int d, int64_t m,
                                  __nv_bfloat16* xn, cudaStream_t st);
cudaError_t ll_attn_prefill(const float* qkv, int m, int pos0, int n_heads, int n_kv, int hd, int max_seq,
                            const __half* cache_k, const __half* cache_v, __nv_bfloat16* ctx, cudaStream_t st);
cudaError_t ll_silu_mul_rows(const float* gu, int64_t m, int ffn, __nv_bfloat16* act, cudaStream_t st);
// fp32 outputs of the two row kernels, for the packed matvec at batches 2..16
cudaError_t ll_resid_rmsnorm_rows_f32(float* h, const float* add, const float* w, float eps, int d, int64_t m, float* xn,
                                      cudaStream_t st);
cudaError_t ll_silu_mul_rows_f32(const float* gu, int64_t m, int ffn, float* act, cudaStream_t st);
cudaError_t ll_add_rows(float* h, const float* add, int64_t total, cudaStream_t st);



}  // namespace qmm

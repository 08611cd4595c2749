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
};

cudaError_t ll_resid_rmsnorm_pack(const float* h_in, const float* add, const float* w, float eps, int d,
                                  uint8_t* packed, float* h_out, const PeerGather& pg, cudaStream_t st);
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


// ---- persistent decoder kernel (llama_mega.cu) ---------------------------------------------------

constexpr int MEGA_WARPS = 24;          // warps per CTA (one CTA per SM)
constexpr int MEGA_RING_BYTES = 6912;   // weight-tile ring of one warp: 3 x 2304 or 2 x 3360 bytes

// One quantized linear as the kernel sees it.
struct MegaLinear {
    const uint8_t* tiles;  // packed weight, [rt][kc] tiles
    float* y;              // output vector [n]
    int n, rt, kc, fmt;
    int wpr;               // warps that share one row tile (divides MEGA_WARPS, >= 2)
    uint32_t tile_bytes;
};

struct MegaLayer {
    const float* attn_norm;
    const float* ffn_norm;
    __half* cache_k;
    __half* cache_v;
};

struct MegaArgs {
    const MegaLinear* lin;    // [4 * n_layers + 1]: qkv, attn_output, gate|up, down per layer, then output
    const MegaLayer* layers;  // [n_layers]
    const float* final_norm;
    const uint8_t* embd;      // raw token_embd payload
    int embd_fmt;
    int n_layers, d_model, n_heads, n_kv, hd, rope_dim, ffn, vocab, max_seq;
    float eps;
    const float* rope_cos;
    const float* rope_sin;
    int* token;       // in: token to process; out: token chosen
    int* pos;         // position of `token`, advanced by one
    int* out_tokens;  // generated tokens so far
    int* out_count;
    float* part;      // [n_heads][nsplit][4 + hd] attention partials: max, sum, -, -, acc[hd]
    int nsplit;
    int* cand;        // [grid][2] arg-max candidates
    unsigned int* sync;  // [0] barrier arrivals, [1] exits; both zero between launches
    int* status;      // set non-zero when a bounded wait ran out
    int kc_max;       // largest kc over the linears (sizes the packed-activation area)
};

// Picks wpr for a linear: the divisor of MEGA_WARPS that minimizes the tiles the busiest warp reads.
int ll_mega_pick_wpr(int rt, int kc, int grid);
// Dynamic shared memory the kernel needs for this model.
size_t ll_mega_smem_bytes(int d_model, int hd, int kc_max, int n_layers);
// One token; cooperative launch of `grid` CTAs (at most one per SM).
cudaError_t ll_mega_decode(const MegaArgs& args, int grid, cudaStream_t st);

}  // namespace qmm

/*
 * litenn_llama.h — C ABI of the LLaMA decoder harness built on the quantized linears of
 * litenn_qmm.h.  It computes what LiteNN's lowered graphs compute
 * (tools/gguf/LLaMABuilder.cpp:502-557 decoder block, :568-668 decode step with explicit
 * KV cache, :682-736 model, :738-759 embedding rows) but keeps every linear weight
 * quantized, keeps a preallocated fp16 KV cache instead of re-lowering a graph per
 * position (LLaMABuilder.cpp:826-872), and adds the greedy loop the reference leaves to
 * the caller (example/gguf/conversion_example.cpp:155-196).
 *
 * Tensor parallelism (no counterpart in LiteNN): every rank holds the row shards of
 * attn_q/k/v, ffn_gate/up and output, and the column shards of attn_output and ffn_down;
 * the partial results of attn_output and of ffn_down are summed over the ranks.  The collective
 * is NCCL, loaded at run time from the library path given to qmm_llama_tp_init; decode can
 * replace it by a direct exchange over peer memory (qmm_llama_tp_export / _import), after which
 * a decoded token launches no collective at all.
 *
 * Conventions are those of litenn_qmm.h: int status codes, qmm_last_error(), streams as void*.
 */
#ifndef LITENN_LLAMA_H
#define LITENN_LLAMA_H

#include "litenn_qmm.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Hyperparameters as parsed by ParseLLaMAHyperparameters (tools/gguf/GGUFImporter.cpp:505-642). */
typedef struct qmm_llama_config {
    int32_t n_layers;
    int32_t d_model;     /* embedding_length */
    int32_t n_heads;     /* attention.head_count */
    int32_t n_kv_heads;  /* attention.head_count_kv */
    int32_t head_dim;
    int32_t ffn;         /* feed_forward_length */
    int32_t vocab;
    int32_t rope_dim;    /* rope.dimension_count (<= head_dim) */
    int32_t max_seq;     /* KV cache capacity in positions */
    int32_t max_prefill; /* largest prompt one qmm_llama_prefill call accepts */
    int32_t tp_rank;
    int32_t tp_size;
    int32_t embd_fmt;    /* block format of token_embd (a QMM_FMT_* value) */
    float rms_eps;
    float rope_theta;
} qmm_llama_config;

typedef struct qmm_llama qmm_llama;

/* Linear weights of one layer, as this rank's shards (qmm_weight_create_shard):
 *   QMM_LL_QKV   rows [q | k | v] of this rank, fused into one [.., d_model] weight
 *   QMM_LL_O     attn_output, K-split
 *   QMM_LL_GU    this rank's rows of gate and up fused into one weight, alternating 8 rows of gate
 *                with the same 8 rows of up (qmm_interleave_gate_up in litenn_qmm.h): the
 *                matvec's epilogue computes silu(gate) * up inside one 16-row tile
 *   QMM_LL_DOWN  ffn_down, K-split
 *   QMM_LL_HEAD  output (lm_head), N-split; layer is ignored
 * Handles are borrowed: they must outlive the model. */
#define QMM_LL_QKV 0
#define QMM_LL_O 1
#define QMM_LL_GU 2
#define QMM_LL_DOWN 3
#define QMM_LL_HEAD 4

/* RMSNorm weights: QMM_LL_ATTN_NORM / QMM_LL_FFN_NORM per layer, QMM_LL_FINAL_NORM once. */
#define QMM_LL_ATTN_NORM 0
#define QMM_LL_FFN_NORM 1
#define QMM_LL_FINAL_NORM 2

int qmm_llama_create(int device, const qmm_llama_config* cfg, qmm_llama** out);
int qmm_llama_destroy(qmm_llama* m);
int qmm_llama_set_weight(qmm_llama* m, int layer, int which, const qmm_weight* w);
int qmm_llama_set_norm(qmm_llama* m, int layer, int which, const float* weights_host);
/* token_embd: the raw ggml payload [vocab, d_model] (host); rows are dequantized on demand. */
int qmm_llama_set_embedding(qmm_llama* m, const void* payload_host, size_t payload_bytes);

/* GGUF files without an output.weight tensor reuse token_embd for the logits
 * (tools/gguf/LLaMABuilder.cpp:719-733).  Packs this rank's rows of the embedding payload as the
 * output weight; the model owns the packed copy.  Use instead of qmm_llama_set_weight(QMM_LL_HEAD). */
int qmm_llama_tie_output(qmm_llama* m, const void* embedding_payload_host, size_t payload_bytes, void* stream);

/* Tensor-parallel set-up.  Rank 0 obtains an id (128 bytes) and hands it to every rank by
 * any host channel; every rank then calls qmm_llama_tp_init with the same id. */
int qmm_llama_tp_unique_id(const char* nccl_library_path, char id_out[128]);
int qmm_llama_tp_init(qmm_llama* m, const char* nccl_library_path, const char id[128]);

/* Optional, after qmm_llama_tp_init: lets decode add the per-block partial sums through
 * peer memory instead of NCCL.  Every rank exports a 128-byte record (a CUDA IPC handle of
 * its receive buffer), the host gathers the records of all ranks in rank order
 * (tp_size * 128 bytes) by any channel, and every rank imports the lot.  From then on the
 * K-split matvecs of decode store their partial sums straight into the peers' buffers over
 * NVLink and, in the same kernel, add the peers' addends in rank order once they have arrived
 * (bounded wait; QMM_E_KERNEL from the next synchronizing call if one never comes), before the
 * residual add and the packing for the next matvec.  The ranks' arg-max winners travel the same way.
 * Ranks must be separate processes (CUDA IPC).  Prefill keeps using NCCL. */
int qmm_llama_tp_export(qmm_llama* m, char handle_out[128]);
int qmm_llama_tp_import(qmm_llama* m, const char* handles, void* stream);

/* Failure detection (no counterpart in LiteNN, whose CUDA backend only checks return codes,
 * src/LiteNN/Device/CUDA.cpp:89-131).
 *   - Every wait of a kernel on a peer's packet is bounded by a number of polls (default 2^21,
 *     about a second); a kernel that gives up sets a status word, later kernels of the model stop
 *     waiting at once, and the next synchronizing call (decode, step_host, prefill) returns
 *     QMM_E_KERNEL.  qmm_llama_reset clears the word.
 *   - While a synchronizing call waits for a stream that carries NCCL collectives it polls
 *     ncclCommGetAsyncError; on an asynchronous error, or when the stream has not drained within
 *     the collective time limit (default 60 s), it calls ncclCommAbort and returns QMM_E_CUDA. */
int qmm_llama_set_wait_limit(qmm_llama* m, unsigned int polls);
int qmm_llama_set_collective_timeout(qmm_llama* m, int milliseconds);
/* Test hook: wires a tensor-parallel model's "peers" to its OWN receive buffer, without NCCL and
 * without other ranks.  Nobody ever fills the peers' slots, so the first decode step runs into the
 * wait limit: this is how the failure path is exercised on one GPU without faulting anything. */
int qmm_llama_tp_loopback(qmm_llama* m);

/* Empties the KV cache (position 0) and the generated-token list.  Tensor-parallel models:
 * a collective, every rank must call it. */
int qmm_llama_reset(qmm_llama* m, void* stream);

/* Runs the prompt (n tokens, host) through the prefill path (bf16 activations, tcgen05 GEMMs),
 * fills the KV cache and produces the first generated token (greedy argmax). */
int qmm_llama_prefill(qmm_llama* m, const int32_t* tokens_host, int n, int32_t* first_token_out, void* stream);

/* Greedy decode: `steps` more tokens, one CUDA graph replay per token (the first decoded token
 * of a model runs eagerly and the graph is captured right after it); synchronizes the stream
 * and copies the tokens to tokens_out_host. */
int qmm_llama_decode(qmm_llama* m, int steps, int32_t* tokens_out_host, void* stream);

/* One decode step driven from the host: copies `token_in` to the device, runs the step,
 * copies the chosen token back and synchronizes — the per-token life of a caller that
 * keeps the sequence on the host. */
int qmm_llama_step_host(qmm_llama* m, int32_t token_in, int32_t* token_out, void* stream);

/* Same work enqueued without synchronizing or copying (for timing with events). */
int qmm_llama_decode_enqueue(qmm_llama* m, int steps, void* stream);

/* Tokens first .. first+count-1 of everything generated since the last reset (the prefill's first
 * token is number 0); synchronizes the stream. */
int qmm_llama_generated_tokens(qmm_llama* m, int first, int count, int32_t* tokens_out_host, void* stream);

/* 1 once the per-token CUDA graph has been captured (after the model's first decoded token). */
int qmm_llama_has_graph(const qmm_llama* m);

/* This rank's logits of the last processed position (vocab / tp_size floats, host). */
int qmm_llama_last_logits(qmm_llama* m, float* logits_host, void* stream);

/*
 * Batched greedy decode: `batch` (1..16) independent sequences share the weights; each has its own fp16
 * KV cache and position.  One step is the decode step of tools/gguf/LLaMABuilder.cpp:568-668 for every
 * sequence at once: the seven linears of a block see the batch as the rows of one skinny product (the
 * packed matvec at batch 2..16, src/LiteNN/Device.h:628-660 with M = batch), attention runs per sequence.
 * One CUDA graph per step.  Tensor-parallel models add the batch's two per-block sums and gather its
 * arg-max candidates with NCCL (qmm_llama_tp_init), whether or not the peer exchange of the
 * single-sequence path has been set up.
 *   qmm_llama_batch_create     allocates the batch's caches and buffers (once per model); at most
 *                              `max_steps` steps can be taken
 *   qmm_llama_batch_prefill    runs the prompt of sequence `seq` (before the first step) and returns its
 *                              first generated token, which becomes the sequence's current token
 *   qmm_llama_batch_decode     `steps` steps; tokens_out_host[step][sequence]
 *   _decode_enqueue / _generated_tokens   the same without / only the copy to the host
 */
int qmm_llama_batch_create(qmm_llama* m, int batch, int max_steps);
int qmm_llama_batch_prefill(qmm_llama* m, int seq, const int32_t* tokens_host, int n, int32_t* first_token_out,
                            void* stream);
int qmm_llama_batch_decode(qmm_llama* m, int steps, int32_t* tokens_out_host, void* stream);
int qmm_llama_batch_decode_enqueue(qmm_llama* m, int steps, void* stream);
int qmm_llama_batch_generated_tokens(qmm_llama* m, int first_step, int steps, int32_t* tokens_out_host, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LITENN_LLAMA_H */

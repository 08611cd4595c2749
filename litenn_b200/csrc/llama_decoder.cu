// LLaMA decoder harness (include/litenn_llama.h): buffers, KV cache, the per-token launch
// sequence captured into a CUDA graph, the prefill sequence, and the tensor-parallel mode: NCCL
// all-reduces in prefill, and in decode either NCCL or the peer-memory exchange built into the
// matvec and commit kernels.  The linears are the quantized kernels of
// qmm_gemv_kernel.cuh / qmm_gemm.cu.
//
// A decoded token is a chain of five kernels per block with no glue kernel between them:
//   qkv matvec          input: packed (h * attn_norm) and the sums of squares of h, both left by the
//                       previous kernel; multiplies its row sums by 1/rms
//   attention           RoPE, KV append, attention over the cache, packs the context
//   attn_output matvec  epilogue: h += result; packs (h * ffn_norm), sums of squares
//   gate|up matvec      rows interleaved gate/up; epilogue: silu(gate) * up, packed for ffn_down (fp32 for
//                       wide models and tensor-parallel shards, whose ffn_down packs its input itself)
//   ffn_down matvec     epilogue: h += result; packs (h * next norm), sums of squares
// (RMSNorm(h) * w = (h * w) / rms(h): packing needs no statistic of the whole row, and the scalar
// 1/rms commutes with the matvec.)  With tensor parallelism the two K-split matvecs also exchange their
// partial sums with the peers inside that epilogue (PeerScatter, qmm_common.cuh); with NCCL sums instead,
// a stand-alone kernel does the residual add and the packing after the all-reduce.
// Batched decode (enqueue_batch_step) is the unfused row form of the same chain.
#include "../../include/litenn_llama.h"

#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "llama_kernels.h"
#include "qmm_internal.h"

using namespace qmm;

namespace {

// ---- NCCL, resolved at run time ----------------------------------------------------------------
struct Id128 {
    char bytes[128];
};
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, /* ncclUniqueId by value: 128 bytes */ Id128, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*CommGetAsyncError)(void*, int*) = nullptr;  // optional
    int (*CommAbort)(void*) = nullptr;                // optional
};
constexpr int NCCL_FLOAT32 = 7, NCCL_INT32 = 2, NCCL_SUM = 0;
constexpr int ARGMAX_CTAS = 16;

NcclApi g_nccl;

int load_nccl(const char* path)
{
    if (g_nccl.lib) {
        return QMM_OK;
    }
    void* lib = dlopen(path && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
        return qmm_internal_fail(QMM_E_UNSUPPORTED, (std::string("cannot load NCCL: ") + dlerror()).c_str());
    }
    NcclApi api;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(lib, "ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(lib, "ncclAllGather"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(dlsym(lib, "ncclCommGetAsyncError"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(dlsym(lib, "ncclCommAbort"));
    if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.AllGather) {
        dlclose(lib);
        return qmm_internal_fail(QMM_E_UNSUPPORTED, "the NCCL library lacks a required symbol");
    }
    api.lib = lib;
    g_nccl = api;
    return QMM_OK;
}

struct Layer {
    const qmm_weight* w[4] = {nullptr, nullptr, nullptr, nullptr};
    float* attn_norm = nullptr;
    float* ffn_norm = nullptr;
    __half* cache_k = nullptr;
    __half* cache_v = nullptr;
};

}  // namespace

struct qmm_llama {
    qmm_llama_config cfg;
    int device = 0;
    int hl = 0, kvl = 0, ffl = 0, vl = 0;  // local heads, kv heads, ffn width, vocab rows
    std::vector<Layer> layers;
    const qmm_weight* head = nullptr;
    qmm_weight* head_owned = nullptr;  // packed from the embedding payload when the output weight is tied
    float* final_norm = nullptr;
    uint8_t* embd = nullptr;
    std::vector<void*> allocs;
    // decode buffers
    float *h = nullptr, *y = nullptr, *qkv = nullptr, *logits = nullptr;
    uint8_t *pk_d = nullptr, *pk_ctx = nullptr;
    float* act_f = nullptr;  // [ffn of this rank] silu(gate) * up, fp32; the ffn_down matvec packs it itself
    uint8_t* pk_act = nullptr;  // the same as packed activations, written by the gate|up matvec (glu_packed)
    bool glu_packed = false;    // d_model <= 4096 and a local ffn width that is a multiple of 32
    double* ss_d = nullptr;  // [d_model / 32] sums of squares of the residual stream
    float *rope_cos = nullptr, *rope_sin = nullptr;
    int *pos = nullptr, *token = nullptr, *out_tokens = nullptr, *out_count = nullptr, *pair = nullptr, *pairs = nullptr;
    // prefill buffers
    float *hr = nullptr, *yr = nullptr, *y2r = nullptr, *qkvr = nullptr, *gur = nullptr;
    __nv_bfloat16 *xn = nullptr, *ctx = nullptr, *act = nullptr;
    int* tokens_dev = nullptr;
    // state
    int host_pos = 0, host_count = 0;
    cudaGraphExec_t graph = nullptr;
    void* comm = nullptr;
    int collective_timeout_ms = 60000;
    // direct peer exchange of the two per-block sums and of the arg-max winners (replaces NCCL in decode):
    // [2][tp][d_model] addend packets {value, exchange number}, then [tp][2] arg-max packets; exported over CUDA IPC
    uint2* xchg = nullptr;
    uint2* peer_xchg[8] = {};  // the same buffer of every peer, mapped here
    bool xchg_ready = false;
    bool loopback = false;     // test hook: the "peer" buffer is this rank's own, nobody fills the peer's slots
    unsigned int spin_limit = 1u << 21;
    int* status = nullptr;     // set non-zero by a kernel whose bounded wait ran out
    // batched decode (qmm_llama_batch_*): `batch` independent sequences share the weights
    int batch = 0, batch_max_steps = 0;
    std::vector<__half*> bcache_k, bcache_v;  // per block: [batch][kv heads][max_seq][head_dim]
    float *bh = nullptr, *bx = nullptr, *bqkv = nullptr, *bctx = nullptr, *by = nullptr, *bgu = nullptr,
          *blogits = nullptr;
    uint8_t* bpk = nullptr;                   // packed activations of the batch (general form)
    int *btok = nullptr, *bpos = nullptr, *bout = nullptr, *bsteps = nullptr, *bpair = nullptr, *bpairs = nullptr;
    std::vector<int> bpos_host, btok_host;
    int bsteps_host = 0;
    cudaGraphExec_t bgraph = nullptr;
    // The peer exchange numbers its arg-max packets by position, which repeats when the sequences of a batch
    // are prefilled one after another: those prefills gather their candidates with NCCL instead.
    bool pick_with_nccl = false;
    // {token, model status, library status} written by the commit kernel into mapped pinned host memory
    int* report_host = nullptr;   // host view
    int* report_dev = nullptr;    // device view of the same words
    int* library_status = nullptr;
};

namespace {

#define LL_CUDA(call)                                                                                   \
    do {                                                                                                \
        cudaError_t e_ = (call);                                                                        \
        if (e_ != cudaSuccess) {                                                                        \
            char buf_[256];                                                                             \
            snprintf(buf_, sizeof buf_, "%s failed: %s", #call, cudaGetErrorString(e_));                \
            return qmm_internal_fail(QMM_E_CUDA, buf_);                                                 \
        }                                                                                               \
    } while (0)

#define LL_QMM(call)         \
    do {                     \
        int rc_ = (call);    \
        if (rc_ != QMM_OK) { \
            return rc_;      \
        }                    \
    } while (0)

#define LL_GUARD(m)                                                           \
    DeviceGuard guard_((m)->device);                                          \
    if (!guard_.ok) {                                                         \
        return qmm_internal_fail(QMM_E_CUDA, cudaGetErrorString(guard_.err)); \
    }

template <typename T>
int dev_alloc(qmm_llama* m, T** p, size_t count)
{
    void* raw = nullptr;
    LL_CUDA(cudaMalloc(&raw, count * sizeof(T) + 256));
    LL_CUDA(cudaMemset(raw, 0, count * sizeof(T) + 256));
    m->allocs.push_back(raw);
    *p = static_cast<T*>(raw);
    return QMM_OK;
}

size_t xchg_packets(const qmm_llama_config& c)
{
    return (size_t)2 * c.tp_size * c.d_model + (size_t)2 * c.tp_size;
}

int all_reduce(qmm_llama* m, float* buf, size_t count, cudaStream_t st)
{
    if (m->cfg.tp_size <= 1) {
        return QMM_OK;
    }
    if (!m->comm) {
        return qmm_internal_fail(QMM_E_INVALID, "tensor-parallel model used before qmm_llama_tp_init");
    }
    if (g_nccl.AllReduce(buf, buf, count, NCCL_FLOAT32, NCCL_SUM, m->comm, st) != 0) {
        return qmm_internal_fail(QMM_E_CUDA, "ncclAllReduce failed");
    }
    return QMM_OK;
}

// cudaStreamSynchronize for a stream that carries collectives: while the stream is busy the
// communicator is polled for an asynchronous error (a peer that died, a network fault), and a
// collective that neither finishes nor fails within the time limit is given up.  Either way the
// communicator is aborted so that the stream drains, and the model refuses further
// tensor-parallel work.
int sync_with_collectives(qmm_llama* m, cudaStream_t st)
{
    if (!m->comm || !g_nccl.CommGetAsyncError) {
        LL_CUDA(cudaStreamSynchronize(st));
        return QMM_OK;
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaStreamQuery(st);
        if (q == cudaSuccess) {
            return QMM_OK;
        }
        if (q != cudaErrorNotReady) {
            LL_CUDA(q);
        }
        int async_err = 0;
        const int rc = g_nccl.CommGetAsyncError(m->comm, &async_err);
        const auto ms =
            std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        const bool late = ms > m->collective_timeout_ms;
        if (rc != 0 || async_err != 0 || late) {
            if (g_nccl.CommAbort) {
                g_nccl.CommAbort(m->comm);
            }
            m->comm = nullptr;
            m->xchg_ready = false;
            char buf[160];
            if (late) {
                snprintf(buf, sizeof buf, "a collective did not finish within %d ms; communicator aborted",
                         m->collective_timeout_ms);
            } else {
                snprintf(buf, sizeof buf, "NCCL reported an asynchronous error (%d); communicator aborted",
                         rc != 0 ? rc : async_err);
            }
            return qmm_internal_fail(QMM_E_CUDA, buf);
        }
    }
}

// Device-to-host read of a result at the end of a call.  A copy into pageable host memory blocks the
// calling thread until the stream has drained, so with a communicator the stream is drained under the
// watch of sync_with_collectives FIRST: a collective that fails or stalls is then reported instead of
// being waited for inside the copy.
int read_back(qmm_llama* m, void* host, const void* dev, size_t bytes, cudaStream_t st)
{
    if (m->comm) {
        LL_QMM(sync_with_collectives(m, st));
    }
    LL_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, st));
    LL_CUDA(cudaStreamSynchronize(st));
    return QMM_OK;
}

// Exchange `site` (0 .. 2*n_layers-1) of a token alternates between two receive buffers: a
// rank can only be one exchange ahead of a peer (it needs the peer's addend to finish its own
// sum), so the buffer it overwrites has been read.
PeerScatter scatter_for(const qmm_llama* m, int site)
{
    PeerScatter ps = {};
    const qmm_llama_config& c = m->cfg;
    const size_t slot = ((size_t)(site & 1) * c.tp_size + c.tp_rank) * c.d_model;
    for (int r = 0; r < c.tp_size; ++r) {
        if (r != c.tp_rank) {
            ps.dst[ps.n_peers++] = m->peer_xchg[r] + slot;
        }
    }
    ps.pos = m->pos;
    ps.sites = 2 * c.n_layers;
    ps.site = site;
    ps.recv = m->xchg + (size_t)(site & 1) * c.tp_size * c.d_model;
    ps.tp_rank = c.tp_rank;
    ps.tp_size = c.tp_size;
    ps.spin_limit = m->spin_limit;
    ps.wait_status = m->status;
    return ps;
}

GemvFuse with_rms(const qmm_llama* m, int mode)
{
    GemvFuse fu = {};
    fu.mode = mode;
    fu.ss_in = m->ss_d;
    fu.ss_count = m->cfg.d_model / 32;
    fu.d_in = m->cfg.d_model;
    fu.eps = m->cfg.rms_eps;
    return fu;
}

// h += W * x summed over the ranks; leaves pk_d = pack(h * norm_w) and ss_d for the matvec that follows.
int linear_resid(qmm_llama* m, const qmm_weight* w, const uint8_t* packed_in, const float* x_f32, const float* norm_w,
                 int site, cudaStream_t st)
{
    const qmm_llama_config& c = m->cfg;
    GemvFuse in = {};  // input side only: fp32 activations are packed by the matvec itself
    in.x_f32 = x_f32;
    if (c.tp_size == 1) {
        GemvFuse fu = in;
        fu.mode = EPI_RESID_PACK;
        fu.h_in = m->h;
        fu.h_out = m->h;
        fu.norm_w = norm_w;
        fu.ss_out = m->ss_d;
        fu.packed_out = m->pk_d;
        return qmm_internal_gemv_fused(w, packed_in, nullptr, nullptr, &fu, st);
    }
    if (m->xchg_ready) {
        // one kernel: partial sums, their exchange over peer memory, the sum over the ranks, residual, packing
        const PeerScatter ps = scatter_for(m, site);
        GemvFuse fu = in;
        fu.mode = EPI_RESID_PACK;
        fu.h_in = m->h;
        fu.h_out = m->h;
        fu.norm_w = norm_w;
        fu.ss_out = m->ss_d;
        fu.packed_out = m->pk_d;
        return qmm_internal_gemv_fused(w, packed_in, nullptr, &ps, &fu, st);
    }
    const PeerGather off = {};
    LL_QMM(qmm_internal_gemv_fused(w, packed_in, m->y, nullptr, &in, st));
    LL_QMM(all_reduce(m, m->y, c.d_model, st));
    LL_CUDA(ll_resid_pack(m->h, m->y, norm_w, c.d_model, m->h, m->pk_d, m->ss_d, off, st));
    return QMM_OK;
}

// pk_d / ss_d -> logits -> this rank's candidates -> winner over the ranks -> token, position, output list
int head_and_pick(qmm_llama* m, cudaStream_t st)
{
    const qmm_llama_config& c = m->cfg;
    const GemvFuse fu = with_rms(m, EPI_STORE);
    LL_QMM(qmm_internal_gemv_fused(m->head, m->pk_d, m->logits, nullptr, &fu, st));
    LL_CUDA(ll_argmax(m->logits, m->vl, m->vl * c.tp_rank, ARGMAX_CTAS, m->pair, 1, 0, st));
    ArgmaxExchange ax = {};
    const int* pairs = m->pair;
    int n_local = ARGMAX_CTAS;
    if (c.tp_size > 1 && m->xchg_ready && !m->pick_with_nccl) {
        const size_t off = (size_t)2 * c.tp_size * c.d_model;
        ax.recv = m->xchg + off;
        for (int r = 0; r < c.tp_size; ++r) {
            ax.peer[r] = m->peer_xchg[r] ? m->peer_xchg[r] + off : nullptr;
        }
        ax.tp_rank = c.tp_rank;
        ax.tp_size = c.tp_size;
        ax.status = m->status;
        ax.spin_limit = m->spin_limit;
    } else if (c.tp_size > 1) {
        if (!m->comm) {
            return qmm_internal_fail(QMM_E_INVALID, "tensor-parallel model used before qmm_llama_tp_init");
        }
        if (g_nccl.AllGather(m->pair, m->pairs, 2 * ARGMAX_CTAS, NCCL_INT32, m->comm, st) != 0) {
            return qmm_internal_fail(QMM_E_CUDA, "ncclAllGather failed");
        }
        pairs = m->pairs;
        n_local = c.tp_size * ARGMAX_CTAS;
    }
    TokenReport report = {};
    report.host = m->report_dev;
    report.model_status = m->status;
    report.library_status = m->library_status;
    LL_CUDA(ll_commit_token(pairs, n_local, ax, m->token, m->pos, m->out_tokens, m->out_count, report, st));
    return QMM_OK;
}

// One token at position *pos: everything reads its inputs from device memory, so the same
// sequence can be replayed from a CUDA graph.
int enqueue_decode_step(qmm_llama* m, cudaStream_t st)
{
    const qmm_llama_config& c = m->cfg;
    LL_CUDA(ll_embed_pack(c.embd_fmt, m->embd, m->token, c.d_model, m->layers[0].attn_norm, m->h, m->pk_d, m->ss_d, st));
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = m->layers[l];
        const GemvFuse rms = with_rms(m, EPI_STORE);
        LL_QMM(qmm_internal_gemv_fused(L.w[QMM_LL_QKV], m->pk_d, m->qkv, nullptr, &rms, st));
        LL_CUDA(ll_attn_fused(m->qkv, m->pos, m->hl, m->kvl, c.head_dim, c.rope_dim, m->rope_cos, m->rope_sin,
                              c.max_seq, L.cache_k, L.cache_v, m->pk_ctx, 1, AttnBatch{}, st));
        LL_QMM(linear_resid(m, L.w[QMM_LL_O], m->pk_ctx, nullptr, L.ffn_norm, 2 * l, st));
        const float* next_norm = l + 1 < c.n_layers ? m->layers[l + 1].attn_norm : m->final_norm;
        if (m->glu_packed) {
            GemvFuse glu = with_rms(m, EPI_SWIGLU_PACK);
            glu.packed_out = m->pk_act;
            LL_QMM(qmm_internal_gemv_fused(L.w[QMM_LL_GU], m->pk_d, nullptr, nullptr, &glu, st));
            LL_QMM(linear_resid(m, L.w[QMM_LL_DOWN], m->pk_act, nullptr, next_norm, 2 * l + 1, st));
        } else {
            const GemvFuse glu = with_rms(m, EPI_SWIGLU);
            LL_QMM(qmm_internal_gemv_fused(L.w[QMM_LL_GU], m->pk_d, m->act_f, nullptr, &glu, st));
            if (m->ffl > 12288) {
                // a long fp32 input is packed once by its own kernel: every CTA of ffn_down packing 100+ KB
                // of activations itself costs more than the extra launch
                LL_QMM(qmm_pack_activations(m->device, m->act_f, 1, m->ffl, m->pk_act, st));
                LL_QMM(linear_resid(m, L.w[QMM_LL_DOWN], m->pk_act, nullptr, next_norm, 2 * l + 1, st));
            } else {
                LL_QMM(linear_resid(m, L.w[QMM_LL_DOWN], nullptr, m->act_f, next_norm, 2 * l + 1, st));
            }
        }
    }
    return head_and_pick(m, st);
}

int check_ready(const qmm_llama* m)
{
    if (!m) {
        return qmm_internal_fail(QMM_E_INVALID, "model handle is null");
    }
    for (const Layer& L : m->layers) {
        for (int i = 0; i < 4; ++i) {
            if (!L.w[i]) {
                return qmm_internal_fail(QMM_E_INVALID, "a layer weight has not been set");
            }
        }
    }
    if (!m->head || !m->embd) {
        return qmm_internal_fail(QMM_E_INVALID, "output weight or embedding has not been set");
    }
    return QMM_OK;
}

// Exchange numbers are a function of the position, so going back to position 0 would make old
// packets look current: every rank clears its receive buffers, then all meet in a collective
// before any rank scatters again.
int rearm_exchange(qmm_llama* m, cudaStream_t st)
{
    if (!m->xchg_ready) {
        return QMM_OK;
    }
    LL_CUDA(cudaMemsetAsync(m->xchg, 0, xchg_packets(m->cfg) * sizeof(uint2), st));
    if (m->loopback) {
        return QMM_OK;
    }
    return all_reduce(m, m->y, 1, st);
}

// After a synchronize: did a kernel of this model give up on a bounded wait for a peer?
int check_status(qmm_llama* m)
{
    int word = 0;
    LL_CUDA(cudaMemcpy(&word, m->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (word != 0) {
        char buf[200];
        snprintf(buf, sizeof buf,
                 "decode: a bounded wait for a peer ran out (status %d: 5 partial sum, 6 arg-max candidate); "
                 "the tokens are invalid until qmm_llama_reset",
                 word);
        return qmm_internal_fail(QMM_E_KERNEL, buf);
    }
    int generic = 0;
    return qmm_kernel_status(m->device, &generic);
}

void drop_graph(qmm_llama* m)
{
    if (m->graph) {
        cudaGraphExecDestroy(m->graph);
        m->graph = nullptr;
    }
    if (m->bgraph) {
        cudaGraphExecDestroy(m->bgraph);
        m->bgraph = nullptr;
    }
}

// One step of `batch` sequences: every sequence's current token -> its next token.  The linears see the
// batch as the rows of one skinny product (packed matvec at batch 2..16); attention, position and cache
// are per sequence.  Unfused on purpose: each stage is the row form of a stage of the batch-1 chain.
int enqueue_batch_step(qmm_llama* m, cudaStream_t st)
{
    const qmm_llama_config& c = m->cfg;
    const int B = m->batch, d = c.d_model, hd = c.head_dim;
    const int qkv_w = (m->hl + 2 * m->kvl) * hd, ctx_w = m->hl * hd;
    auto linear = [&](const qmm_weight* w, const float* x, int64_t k, float* y) -> int {
        LL_QMM(qmm_pack_activations(m->device, x, B, k, m->bpk, st));
        return qmm_gemv_packed(w, m->bpk, y, B, st);
    };
    LL_CUDA(ll_embed_rows(c.embd_fmt, m->embd, m->btok, B, d, m->bh, st));
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = m->layers[l];
        LL_CUDA(ll_resid_rmsnorm_rows_f32(m->bh, l == 0 ? nullptr : m->by, L.attn_norm, c.rms_eps, d, B, m->bx, st));
        LL_QMM(linear(L.w[QMM_LL_QKV], m->bx, d, m->bqkv));
        AttnBatch ab = {};
        ab.qkv_stride = qkv_w;
        ab.cache_stride = (int64_t)m->kvl * c.max_seq * hd;
        ab.ctx = m->bctx;
        ab.ctx_stride = ctx_w;
        LL_CUDA(ll_attn_fused(m->bqkv, m->bpos, m->hl, m->kvl, hd, c.rope_dim, m->rope_cos, m->rope_sin, c.max_seq,
                              m->bcache_k[l], m->bcache_v[l], nullptr, B, ab, st));
        LL_QMM(linear(L.w[QMM_LL_O], m->bctx, ctx_w, m->by));
        LL_QMM(all_reduce(m, m->by, (size_t)B * d, st));
        LL_CUDA(ll_resid_rmsnorm_rows_f32(m->bh, m->by, L.ffn_norm, c.rms_eps, d, B, m->bx, st));
        LL_QMM(linear(L.w[QMM_LL_GU], m->bx, d, m->bgu));
        LL_CUDA(ll_silu_mul_rows_f32(m->bgu, B, m->ffl, m->bx, st));
        LL_QMM(linear(L.w[QMM_LL_DOWN], m->bx, m->ffl, m->by));
        LL_QMM(all_reduce(m, m->by, (size_t)B * d, st));
    }
    LL_CUDA(ll_resid_rmsnorm_rows_f32(m->bh, m->by, m->final_norm, c.rms_eps, d, B, m->bx, st));
    LL_QMM(linear(m->head, m->bx, d, m->blogits));
    LL_CUDA(ll_argmax(m->blogits, m->vl, m->vl * c.tp_rank, ARGMAX_CTAS, m->bpair, B, m->vl, st));
    const int* pairs = m->bpair;
    if (c.tp_size > 1) {
        if (!m->comm) {
            return qmm_internal_fail(QMM_E_INVALID, "tensor-parallel model used before qmm_llama_tp_init");
        }
        if (g_nccl.AllGather(m->bpair, m->bpairs, (size_t)B * 2 * ARGMAX_CTAS, NCCL_INT32, m->comm, st) != 0) {
            return qmm_internal_fail(QMM_E_CUDA, "ncclAllGather failed");
        }
        pairs = m->bpairs;
    }
    LL_CUDA(ll_commit_batch(pairs, ARGMAX_CTAS, c.tp_size, B, m->btok, m->bpos, m->bout, m->bsteps, st));
    return QMM_OK;
}

}  // namespace

extern "C" {

int qmm_llama_create(int device, const qmm_llama_config* cfg, qmm_llama** out)
{
    if (!cfg || !out) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_create: null argument");
    }
    *out = nullptr;
    const qmm_llama_config& c = *cfg;
    if (c.n_layers < 1 || c.d_model < 1 || c.n_heads < 1 || c.n_kv_heads < 1 || (c.head_dim != 64 && c.head_dim != 128) ||
        c.rope_dim > c.head_dim || c.rope_dim < 2 || (c.rope_dim % 2) != 0 || c.tp_size < 1 || c.tp_size > 8 ||
        c.tp_rank < 0 || c.tp_rank >= c.tp_size || c.max_seq < 1 || c.vocab < 1 || c.ffn < 1) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_create: invalid hyperparameters");
    }
    if (c.n_heads % c.n_kv_heads != 0 || c.n_heads % c.tp_size != 0 || c.n_kv_heads % c.tp_size != 0 ||
        c.ffn % c.tp_size != 0 || c.vocab % c.tp_size != 0) {
        return qmm_internal_fail(QMM_E_INVALID,
                                 "heads, kv heads, ffn width and vocabulary must divide over the tensor-parallel ranks");
    }
    if (c.d_model % 32 != 0 || (c.ffn / c.tp_size) % 32 != 0) {
        return qmm_internal_fail(QMM_E_INVALID,
                                 "d_model and this rank's ffn width must be multiples of 32 (the quantization block)");
    }
    if (block_elems(c.embd_fmt) == 0 || c.d_model % block_elems(c.embd_fmt) != 0) {
        return qmm_internal_fail(QMM_E_INVALID, "embedding format or width not supported");
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return qmm_internal_fail(QMM_E_CUDA, cudaGetErrorString(guard.err));
    }
    qmm_llama* m = new qmm_llama();
    m->cfg = c;
    m->device = device;
    m->hl = c.n_heads / c.tp_size;
    m->kvl = c.n_kv_heads / c.tp_size;
    m->ffl = c.ffn / c.tp_size;
    m->vl = c.vocab / c.tp_size;
    m->layers.resize(c.n_layers);
    const int d = c.d_model, hd = c.head_dim;
    const int qkv_w = (m->hl + 2 * m->kvl) * hd;
    size_t pk = 0;
    int rc = QMM_OK;
    const std::vector<float> ones((size_t)d, 1.0f);  // norm weights are 1 until qmm_llama_set_norm
    auto alloc_norm = [&](float** p) -> int {
        LL_QMM(dev_alloc(m, p, d));
        LL_CUDA(cudaMemcpy(*p, ones.data(), (size_t)d * sizeof(float), cudaMemcpyHostToDevice));
        return QMM_OK;
    };
#define LL_TRY(x)                \
    if (rc == QMM_OK) {          \
        rc = (x);                \
    }
    LL_TRY(dev_alloc(m, &m->h, d));
    LL_TRY(dev_alloc(m, &m->status, 1));
    LL_TRY(qmm_internal_status_word(device, &m->library_status));
    {
        void* host = nullptr;
        void* dev = nullptr;
        if (cudaHostAlloc(&host, 4 * sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
            cudaHostGetDevicePointer(&dev, host, 0) != cudaSuccess) {
            cudaGetLastError();
            if (host) {
                cudaFreeHost(host);
            }
            host = nullptr;  // without it every call reads the results with copies, as before
            dev = nullptr;
        } else {
            memset(host, 0, 4 * sizeof(int));
        }
        m->report_host = static_cast<int*>(host);
        m->report_dev = static_cast<int*>(dev);
    }
    LL_TRY(dev_alloc(m, &m->y, d));
    LL_TRY(dev_alloc(m, &m->qkv, qkv_w));
    LL_TRY(dev_alloc(m, &m->logits, m->vl));
    LL_TRY(dev_alloc(m, &m->ss_d, d / 32));
    LL_TRY(qmm_packed_activation_bytes(d, 1, &pk));
    LL_TRY(dev_alloc(m, &m->pk_d, pk));
    LL_TRY(qmm_packed_activation_bytes((int64_t)m->hl * hd, 1, &pk));
    LL_TRY(dev_alloc(m, &m->pk_ctx, pk));
    LL_TRY(dev_alloc(m, &m->act_f, (size_t)m->ffl));
    LL_TRY(dev_alloc(m, &m->pk_act, xpack1_bytes((m->ffl + 255) / 256)));  // zeroed: blocks past ffl stay zero
    // The packed SwiGLU form gives a CTA four row tiles with two warps each; beyond 16 chunks per row a warp
    // would walk too many tiles one after the other, and the fp32 form with one tile per CTA and eight warps
    // per tile is used.  Tensor-parallel shards take the packed form too: fewer groups of four tiles per rank,
    // but ffn_down no longer packs its input in every CTA (7B shape: 942 -> 985 tok/s at 2 ranks, 1014 -> 1069
    // at 4).
    m->glu_packed = d <= 4096 && m->ffl % 32 == 0 && getenv("QMM_LL_GLU_F32") == nullptr;
    LL_TRY(dev_alloc(m, &m->rope_cos, (size_t)c.max_seq * (c.rope_dim / 2)));
    LL_TRY(dev_alloc(m, &m->rope_sin, (size_t)c.max_seq * (c.rope_dim / 2)));
    LL_TRY(dev_alloc(m, &m->pos, 1));
    LL_TRY(dev_alloc(m, &m->token, 1));
    LL_TRY(dev_alloc(m, &m->out_tokens, (size_t)c.max_seq + 8));
    LL_TRY(dev_alloc(m, &m->out_count, 1));
    LL_TRY(dev_alloc(m, &m->pair, 2 * ARGMAX_CTAS));
    LL_TRY(dev_alloc(m, &m->pairs, (size_t)2 * ARGMAX_CTAS * c.tp_size));
    LL_TRY(alloc_norm(&m->final_norm));
    for (int l = 0; l < c.n_layers && rc == QMM_OK; ++l) {
        LL_TRY(alloc_norm(&m->layers[l].attn_norm));
        LL_TRY(alloc_norm(&m->layers[l].ffn_norm));
        LL_TRY(dev_alloc(m, &m->layers[l].cache_k, (size_t)m->kvl * c.max_seq * hd));
        LL_TRY(dev_alloc(m, &m->layers[l].cache_v, (size_t)m->kvl * c.max_seq * hd));
    }
    const int mp = c.max_prefill;
    if (mp > 0) {
        LL_TRY(dev_alloc(m, &m->hr, (size_t)mp * d));
        LL_TRY(dev_alloc(m, &m->yr, (size_t)mp * d));
        LL_TRY(dev_alloc(m, &m->y2r, (size_t)mp * d));
        LL_TRY(dev_alloc(m, &m->qkvr, (size_t)mp * qkv_w));
        LL_TRY(dev_alloc(m, &m->gur, (size_t)mp * 2 * m->ffl));
        LL_TRY(dev_alloc(m, &m->xn, (size_t)mp * d));
        LL_TRY(dev_alloc(m, &m->ctx, (size_t)mp * m->hl * hd));
        LL_TRY(dev_alloc(m, &m->act, (size_t)mp * m->ffl));
        LL_TRY(dev_alloc(m, &m->tokens_dev, mp));
    }
#undef LL_TRY
    if (rc == QMM_OK) {
        cudaError_t e = ll_rope_tables(c.max_seq, c.rope_dim, (double)c.rope_theta, m->rope_cos, m->rope_sin, nullptr);
        if (e == cudaSuccess) {
            e = cudaDeviceSynchronize();
        }
        if (e != cudaSuccess) {
            rc = qmm_internal_fail(QMM_E_CUDA, cudaGetErrorString(e));
        }
    }
    if (rc != QMM_OK) {
        qmm_llama_destroy(m);
        return rc;
    }
    // allocate the per-device kernel status word now: it must exist before any stream capture
    int st_word = 0;
    rc = qmm_kernel_status(device, &st_word);
    if (rc != QMM_OK) {
        qmm_llama_destroy(m);
        return rc;
    }
    *out = m;
    return QMM_OK;
}

int qmm_llama_destroy(qmm_llama* m)
{
    if (!m) {
        return QMM_OK;
    }
    DeviceGuard guard(m->device);
    drop_graph(m);
    if (m->comm && g_nccl.CommDestroy) {
        g_nccl.CommDestroy(m->comm);
    }
    if (!m->loopback) {
        for (uint2* p : m->peer_xchg) {
            if (p) {
                cudaIpcCloseMemHandle(p);
            }
        }
    }
    if (m->head_owned) {
        qmm_weight_destroy(m->head_owned);
    }
    for (void* p : m->allocs) {
        cudaFree(p);
    }
    if (m->report_host) {
        cudaFreeHost(m->report_host);
    }
    delete m;
    return QMM_OK;
}

int qmm_llama_set_weight(qmm_llama* m, int layer, int which, const qmm_weight* w)
{
    if (!m || !w) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_weight: null argument");
    }
    qmm_weight_info info;
    LL_QMM(qmm_weight_get_info(w, &info));
    const qmm_llama_config& c = m->cfg;
    const int hd = c.head_dim;
    int64_t want_n = 0, want_k = 0;
    switch (which) {
    case QMM_LL_QKV: want_n = (int64_t)(m->hl + 2 * m->kvl) * hd; want_k = c.d_model; break;
    case QMM_LL_O: want_n = c.d_model; want_k = (int64_t)m->hl * hd; break;
    case QMM_LL_GU: want_n = 2 * (int64_t)m->ffl; want_k = c.d_model; break;
    case QMM_LL_DOWN: want_n = c.d_model; want_k = m->ffl; break;
    case QMM_LL_HEAD: want_n = m->vl; want_k = c.d_model; break;
    default: return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_weight: unknown weight kind");
    }
    if (info.n != want_n || info.k != want_k || info.device != m->device) {
        char buf[200];
        snprintf(buf, sizeof buf, "weight kind %d must be [%lld, %lld] on device %d, got [%lld, %lld] on device %d", which,
                 (long long)want_n, (long long)want_k, m->device, (long long)info.n, (long long)info.k, info.device);
        return qmm_internal_fail(QMM_E_INVALID, buf);
    }
    if (which == QMM_LL_HEAD) {
        m->head = w;
    } else {
        if (layer < 0 || layer >= c.n_layers) {
            return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_weight: layer out of range");
        }
        m->layers[layer].w[which] = w;
    }
    drop_graph(m);
    return QMM_OK;
}

int qmm_llama_set_norm(qmm_llama* m, int layer, int which, const float* weights_host)
{
    if (!m || !weights_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_norm: null argument");
    }
    float* dst = nullptr;
    if (which == QMM_LL_FINAL_NORM) {
        dst = m->final_norm;
    } else if (layer >= 0 && layer < m->cfg.n_layers && (which == QMM_LL_ATTN_NORM || which == QMM_LL_FFN_NORM)) {
        dst = which == QMM_LL_ATTN_NORM ? m->layers[layer].attn_norm : m->layers[layer].ffn_norm;
    } else {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_norm: layer or kind out of range");
    }
    LL_GUARD(m);
    LL_CUDA(cudaMemcpy(dst, weights_host, (size_t)m->cfg.d_model * sizeof(float), cudaMemcpyHostToDevice));
    return QMM_OK;
}

int qmm_llama_set_embedding(qmm_llama* m, const void* payload_host, size_t payload_bytes)
{
    if (!m || !payload_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_embedding: null argument");
    }
    const qmm_llama_config& c = m->cfg;
    const size_t want = (size_t)c.vocab * (c.d_model / block_elems(c.embd_fmt)) * block_bytes(c.embd_fmt);
    if (payload_bytes != want) {
        return qmm_internal_fail(QMM_E_INVALID, "embedding payload byte count does not match [vocab, d_model]");
    }
    LL_GUARD(m);
    if (!m->embd) {
        LL_QMM(dev_alloc(m, &m->embd, payload_bytes));
    }
    LL_CUDA(cudaMemcpy(m->embd, payload_host, payload_bytes, cudaMemcpyHostToDevice));
    return QMM_OK;
}

int qmm_llama_tie_output(qmm_llama* m, const void* embedding_payload_host, size_t payload_bytes, void* stream)
{
    if (!m || !embedding_payload_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_tie_output: null argument");
    }
    const qmm_llama_config& c = m->cfg;
    qmm_weight* w = nullptr;
    LL_QMM(qmm_weight_create_shard(m->device, c.embd_fmt, embedding_payload_host, payload_bytes, 0, c.vocab, c.d_model,
                                   c.tp_size > 1 ? QMM_SPLIT_N : QMM_SPLIT_NONE, c.tp_rank, c.tp_size, stream, &w));
    if (m->head_owned) {
        qmm_weight_destroy(m->head_owned);
    }
    m->head_owned = w;
    m->head = w;
    drop_graph(m);
    return QMM_OK;
}

int qmm_interleave_gate_up(int fmt, const void* gate_host, const void* up_host, int64_t n_each, int64_t k, void* out_host)
{
    if (!gate_host || !up_host || !out_host || block_elems(fmt) == 0 || n_each < 8 || n_each % 8 != 0 || k < 1 ||
        k % block_elems(fmt) != 0) {
        return qmm_internal_fail(QMM_E_INVALID,
                                 "qmm_interleave_gate_up: rows must come in groups of 8 and k in whole blocks");
    }
    const size_t grp = (size_t)8 * (k / block_elems(fmt)) * block_bytes(fmt);  // bytes of 8 rows
    const uint8_t* g = static_cast<const uint8_t*>(gate_host);
    const uint8_t* u = static_cast<const uint8_t*>(up_host);
    uint8_t* o = static_cast<uint8_t*>(out_host);
    for (int64_t i = 0; i < n_each / 8; ++i) {
        memcpy(o + (size_t)(2 * i) * grp, g + (size_t)i * grp, grp);
        memcpy(o + (size_t)(2 * i + 1) * grp, u + (size_t)i * grp, grp);
    }
    return QMM_OK;
}

int qmm_llama_tp_unique_id(const char* nccl_library_path, char id_out[128])
{
    LL_QMM(load_nccl(nccl_library_path));
    if (g_nccl.GetUniqueId(id_out) != 0) {
        return qmm_internal_fail(QMM_E_CUDA, "ncclGetUniqueId failed");
    }
    return QMM_OK;
}

int qmm_llama_tp_init(qmm_llama* m, const char* nccl_library_path, const char id[128])
{
    if (!m || !id) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_tp_init: null argument");
    }
    if (m->cfg.tp_size <= 1) {
        return QMM_OK;
    }
    LL_QMM(load_nccl(nccl_library_path));
    LL_GUARD(m);
    Id128 uid;
    memcpy(uid.bytes, id, 128);
    if (g_nccl.CommInitRank(&m->comm, m->cfg.tp_size, uid, m->cfg.tp_rank) != 0) {
        return qmm_internal_fail(QMM_E_CUDA, "ncclCommInitRank failed");
    }
    return QMM_OK;
}

int qmm_llama_set_collective_timeout(qmm_llama* m, int milliseconds)
{
    if (!m || milliseconds < 1) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_collective_timeout: invalid argument");
    }
    m->collective_timeout_ms = milliseconds;
    return QMM_OK;
}

int qmm_llama_set_wait_limit(qmm_llama* m, unsigned int polls)
{
    if (!m || polls < 1) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_wait_limit: invalid argument");
    }
    m->spin_limit = polls;
    drop_graph(m);  // the limit is a kernel argument recorded in the graph
    return QMM_OK;
}

int qmm_llama_tp_export(qmm_llama* m, char handle_out[128])
{
    if (!m || !handle_out) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_tp_export: null argument");
    }
    memset(handle_out, 0, 128);
    if (m->cfg.tp_size <= 1) {
        return QMM_OK;
    }
    LL_GUARD(m);
    if (!m->xchg) {
        LL_QMM(dev_alloc(m, &m->xchg, xchg_packets(m->cfg)));
    }
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) <= 128, "IPC handle larger than the exchange record");
    LL_CUDA(cudaIpcGetMemHandle(&h, m->xchg));
    memcpy(handle_out, &h, sizeof(h));
    return QMM_OK;
}

int qmm_llama_tp_import(qmm_llama* m, const char* handles, void* stream)
{
    if (!m || !handles) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_tp_import: null argument");
    }
    const qmm_llama_config& c = m->cfg;
    if (c.tp_size <= 1) {
        return QMM_OK;
    }
    if (!m->xchg || !m->comm) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_tp_import: call qmm_llama_tp_init and qmm_llama_tp_export first");
    }
    LL_GUARD(m);
    for (int r = 0; r < c.tp_size; ++r) {
        if (r == c.tp_rank || m->peer_xchg[r]) {
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 128, sizeof(h));
        void* p = nullptr;
        LL_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        m->peer_xchg[r] = static_cast<uint2*>(p);
    }
    m->xchg_ready = true;
    drop_graph(m);  // a graph captured earlier still holds the all-reduce form
    return rearm_exchange(m, static_cast<cudaStream_t>(stream));
}

int qmm_llama_tp_loopback(qmm_llama* m)
{
    if (!m || m->cfg.tp_size <= 1 || m->comm || m->xchg_ready) {
        return qmm_internal_fail(QMM_E_INVALID,
                                 "qmm_llama_tp_loopback: needs a tensor-parallel model without a communicator");
    }
    LL_GUARD(m);
    if (!m->xchg) {
        LL_QMM(dev_alloc(m, &m->xchg, xchg_packets(m->cfg)));
    }
    for (int r = 0; r < m->cfg.tp_size; ++r) {
        m->peer_xchg[r] = r == m->cfg.tp_rank ? nullptr : m->xchg;
    }
    m->loopback = true;
    m->xchg_ready = true;
    drop_graph(m);
    return QMM_OK;
}

int qmm_llama_reset(qmm_llama* m, void* stream)
{
    if (!m) {
        return qmm_internal_fail(QMM_E_INVALID, "model handle is null");
    }
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_CUDA(cudaMemsetAsync(m->pos, 0, sizeof(int), st));
    LL_CUDA(cudaMemsetAsync(m->out_count, 0, sizeof(int), st));
    LL_CUDA(cudaMemsetAsync(m->status, 0, sizeof(int), st));
    if (m->batch) {  // the batch's sequences start over as well (their caches are simply overwritten)
        LL_CUDA(cudaMemsetAsync(m->bpos, 0, (size_t)m->batch * sizeof(int), st));
        LL_CUDA(cudaMemsetAsync(m->btok, 0, (size_t)m->batch * sizeof(int), st));
        LL_CUDA(cudaMemsetAsync(m->bsteps, 0, sizeof(int), st));
        std::fill(m->bpos_host.begin(), m->bpos_host.end(), 0);
        m->bsteps_host = 0;
    }
    LL_QMM(rearm_exchange(m, st));
    LL_QMM(sync_with_collectives(m, st));
    m->host_pos = 0;
    m->host_count = 0;
    return QMM_OK;
}

int qmm_llama_prefill(qmm_llama* m, const int32_t* tokens_host, int n, int32_t* first_token_out, void* stream)
{
    LL_QMM(check_ready(m));
    const qmm_llama_config& c = m->cfg;
    if (!tokens_host || n < 1 || n > c.max_prefill || m->host_pos + n > c.max_seq) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_prefill: prompt length outside 1..max_prefill or cache full");
    }
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int d = c.d_model, hd = c.head_dim;
    const int pos0 = m->host_pos;
    LL_CUDA(cudaMemcpyAsync(m->tokens_dev, tokens_host, (size_t)n * sizeof(int), cudaMemcpyHostToDevice, st));
    LL_CUDA(ll_embed_rows(c.embd_fmt, m->embd, m->tokens_dev, n, d, m->hr, st));
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = m->layers[l];
        LL_CUDA(ll_resid_rmsnorm_rows(m->hr, l == 0 ? nullptr : m->y2r, L.attn_norm, c.rms_eps, d, n, m->xn, st));
        LL_QMM(qmm_gemm_bf16(L.w[QMM_LL_QKV], m->xn, m->qkvr, n, QMM_OUT_F32, st));
        LL_CUDA(ll_rope_kv(m->qkvr, m->pos, 0, n, m->hl, m->kvl, hd, c.rope_dim, m->rope_cos, m->rope_sin, c.max_seq,
                           L.cache_k, L.cache_v, st));
        LL_CUDA(ll_attn_prefill(m->qkvr, n, pos0, m->hl, m->kvl, hd, c.max_seq, L.cache_k, L.cache_v, m->ctx, st));
        LL_QMM(qmm_gemm_bf16(L.w[QMM_LL_O], m->ctx, m->yr, n, QMM_OUT_F32, st));
        LL_QMM(all_reduce(m, m->yr, (size_t)n * d, st));
        LL_CUDA(ll_resid_rmsnorm_rows(m->hr, m->yr, L.ffn_norm, c.rms_eps, d, n, m->xn, st));
        LL_QMM(qmm_gemm_bf16(L.w[QMM_LL_GU], m->xn, m->gur, n, QMM_OUT_F32, st));
        LL_CUDA(ll_silu_mul_rows(m->gur, n, m->ffl, m->act, st));
        LL_QMM(qmm_gemm_bf16(L.w[QMM_LL_DOWN], m->act, m->y2r, n, QMM_OUT_F32, st));
        LL_QMM(all_reduce(m, m->y2r, (size_t)n * d, st));
    }
    // the last prompt position produces the first generated token
    const int last_pos = pos0 + n - 1;
    LL_CUDA(cudaMemcpyAsync(m->pos, &last_pos, sizeof(int), cudaMemcpyHostToDevice, st));
    const PeerGather off = {};
    LL_CUDA(ll_resid_pack(m->hr + (size_t)(n - 1) * d, m->y2r + (size_t)(n - 1) * d, m->final_norm, d, nullptr, m->pk_d,
                          m->ss_d, off, st));
    LL_QMM(head_and_pick(m, st));
    int32_t tok = 0;
    LL_QMM(read_back(m, &tok, m->token, sizeof(int), st));
    LL_QMM(check_status(m));
    m->host_pos = pos0 + n;
    m->host_count += 1;
    if (first_token_out) {
        *first_token_out = tok;
    }
    return QMM_OK;
}

int qmm_llama_decode_enqueue(qmm_llama* m, int steps, void* stream)
{
    LL_QMM(check_ready(m));
    if (steps < 1 || m->host_pos + steps > m->cfg.max_seq) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_decode: step count outside the KV cache capacity");
    }
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!m->graph) {
        if (st == nullptr) {
            return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_decode needs a non-default stream (graph capture)");
        }
        // The first token runs eagerly (it also performs every kernel's one-time set-up outside
        // a capture); the same sequence is then captured once and replayed for all later tokens,
        // also when this call asked for one token only.
        LL_QMM(enqueue_decode_step(m, st));
        m->host_pos += 1;
        m->host_count += 1;
        steps -= 1;
        cudaGraph_t g = nullptr;
        LL_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_decode_step(m, st);
        const cudaError_t e = cudaStreamEndCapture(st, &g);
        if (rc != QMM_OK) {
            if (g) {
                cudaGraphDestroy(g);
            }
            return rc;
        }
        LL_CUDA(e);
        LL_CUDA(cudaGraphInstantiate(&m->graph, g, 0));
        cudaGraphDestroy(g);
    }
    for (int s = 0; s < steps; ++s) {
        LL_CUDA(cudaGraphLaunch(m->graph, st));
    }
    m->host_pos += steps;
    m->host_count += steps;
    return QMM_OK;
}

int qmm_llama_decode(qmm_llama* m, int steps, int32_t* tokens_out_host, void* stream)
{
    if (!tokens_out_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_decode: output pointer is null");
    }
    const int first = m ? m->host_count : 0;
    LL_QMM(qmm_llama_decode_enqueue(m, steps, stream));
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_QMM(read_back(m, tokens_out_host, m->out_tokens + first, (size_t)steps * sizeof(int), st));
    return check_status(m);
}

int qmm_llama_step_host(qmm_llama* m, int32_t token_in, int32_t* token_out, void* stream)
{
    if (!m || !token_out) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_step_host: null argument");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_GUARD(m);
    LL_CUDA(cudaMemcpyAsync(m->token, &token_in, sizeof(int), cudaMemcpyHostToDevice, st));
    LL_QMM(qmm_llama_decode_enqueue(m, 1, stream));
    if (m->report_host) {
        // the commit kernel left the token and both status words in host-visible memory: one drain, no copies
        LL_QMM(sync_with_collectives(m, st));
        *token_out = m->report_host[0];
        if (m->report_host[1] == 0 && m->report_host[2] == 0) {
            return QMM_OK;
        }
        return check_status(m);  // builds the error from the device-side words
    }
    LL_QMM(read_back(m, token_out, m->token, sizeof(int), st));
    return check_status(m);
}

int qmm_llama_generated_tokens(qmm_llama* m, int first, int count, int32_t* tokens_out_host, void* stream)
{
    if (!m || !tokens_out_host || first < 0 || count < 0 || first + count > m->host_count) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_generated_tokens: range outside the tokens generated so far");
    }
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_QMM(read_back(m, tokens_out_host, m->out_tokens + first, (size_t)count * sizeof(int), st));
    return check_status(m);
}

int qmm_llama_has_graph(const qmm_llama* m)
{
    return m && m->graph ? 1 : 0;
}

// ---- batched decode ---------------------------------------------------------------------------------

int qmm_llama_batch_create(qmm_llama* m, int batch, int max_steps)
{
    LL_QMM(check_ready(m));
    if (m->batch != 0) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_create: the model already has a batch");
    }
    if (batch < 1 || batch > QMM_GEMV_MAX_BATCH || max_steps < 1) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_create: batch outside 1..16 or no steps");
    }
    LL_GUARD(m);
    const qmm_llama_config& c = m->cfg;
    const size_t B = (size_t)batch, d = (size_t)c.d_model, hd = (size_t)c.head_dim;
    const size_t qkv_w = (size_t)(m->hl + 2 * m->kvl) * hd, ctx_w = (size_t)m->hl * hd;
    const size_t widest = std::max(std::max(d, ctx_w), (size_t)m->ffl);
    size_t pk = 0;
    LL_QMM(qmm_packed_activation_bytes((int64_t)widest, batch, &pk));
    LL_QMM(dev_alloc(m, &m->bh, B * d));
    LL_QMM(dev_alloc(m, &m->bx, B * widest));
    LL_QMM(dev_alloc(m, &m->bqkv, B * qkv_w));
    LL_QMM(dev_alloc(m, &m->bctx, B * ctx_w));
    LL_QMM(dev_alloc(m, &m->by, B * d));
    LL_QMM(dev_alloc(m, &m->bgu, B * 2 * (size_t)m->ffl));
    LL_QMM(dev_alloc(m, &m->blogits, B * (size_t)m->vl));
    LL_QMM(dev_alloc(m, &m->bpk, pk));
    LL_QMM(dev_alloc(m, &m->btok, B));
    LL_QMM(dev_alloc(m, &m->bpos, B));
    LL_QMM(dev_alloc(m, &m->bout, B * (size_t)max_steps));
    LL_QMM(dev_alloc(m, &m->bsteps, 1));
    LL_QMM(dev_alloc(m, &m->bpair, B * 2 * ARGMAX_CTAS));
    LL_QMM(dev_alloc(m, &m->bpairs, B * 2 * ARGMAX_CTAS * (size_t)c.tp_size));
    m->bcache_k.assign(c.n_layers, nullptr);
    m->bcache_v.assign(c.n_layers, nullptr);
    for (int l = 0; l < c.n_layers; ++l) {
        LL_QMM(dev_alloc(m, &m->bcache_k[l], B * (size_t)m->kvl * c.max_seq * hd));
        LL_QMM(dev_alloc(m, &m->bcache_v[l], B * (size_t)m->kvl * c.max_seq * hd));
    }
    m->bpos_host.assign(batch, 0);
    m->btok_host.assign(batch, 0);
    m->bsteps_host = 0;
    m->batch_max_steps = max_steps;
    m->batch = batch;
    return QMM_OK;
}

int qmm_llama_batch_prefill(qmm_llama* m, int seq, const int32_t* tokens_host, int n, int32_t* first_token_out,
                            void* stream)
{
    if (!m || m->batch == 0 || seq < 0 || seq >= m->batch) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_prefill: no batch or sequence index outside it");
    }
    if (m->bpos_host[seq] != 0 || m->bsteps_host != 0) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_prefill: the sequence already holds a prompt");
    }
    // The single-sequence prefill runs on this sequence's caches; the single sequence's own decode state
    // (position, token count, current token; the list entry the prefill appends lies beyond the count) is
    // put back afterwards, so batch and single sequence can be used side by side.
    const size_t stride = (size_t)m->kvl * m->cfg.max_seq * m->cfg.head_dim;
    std::vector<std::pair<__half*, __half*>> own(m->layers.size());
    for (size_t l = 0; l < m->layers.size(); ++l) {
        own[l] = {m->layers[l].cache_k, m->layers[l].cache_v};
        m->layers[l].cache_k = m->bcache_k[l] + (size_t)seq * stride;
        m->layers[l].cache_v = m->bcache_v[l] + (size_t)seq * stride;
    }
    const int saved_pos = m->host_pos, saved_count = m->host_count;
    int saved_dev[3] = {0, 0, 0};  // device-side position, token count and current token of the single sequence
    {
        LL_GUARD(m);
        cudaStream_t st0 = static_cast<cudaStream_t>(stream);
        LL_QMM(read_back(m, &saved_dev[0], m->pos, sizeof(int), st0));
        LL_QMM(read_back(m, &saved_dev[1], m->out_count, sizeof(int), st0));
        LL_QMM(read_back(m, &saved_dev[2], m->token, sizeof(int), st0));
        // the prefill kernels take their first position from the device-side counter
        LL_CUDA(cudaMemsetAsync(m->pos, 0, sizeof(int), st0));
    }
    m->host_pos = 0;
    m->pick_with_nccl = true;
    int32_t first = 0;
    const int rc = qmm_llama_prefill(m, tokens_host, n, &first, stream);
    m->pick_with_nccl = false;
    for (size_t l = 0; l < m->layers.size(); ++l) {
        m->layers[l].cache_k = own[l].first;
        m->layers[l].cache_v = own[l].second;
    }
    m->host_pos = saved_pos;
    m->host_count = saved_count;
    LL_QMM(rc);
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_CUDA(cudaMemcpyAsync(m->pos, &saved_dev[0], sizeof(int), cudaMemcpyHostToDevice, st));
    LL_CUDA(cudaMemcpyAsync(m->out_count, &saved_dev[1], sizeof(int), cudaMemcpyHostToDevice, st));
    LL_CUDA(cudaMemcpyAsync(m->token, &saved_dev[2], sizeof(int), cudaMemcpyHostToDevice, st));
    m->bpos_host[seq] = n;
    m->btok_host[seq] = first;
    LL_CUDA(cudaMemcpyAsync(m->bpos + seq, &m->bpos_host[seq], sizeof(int), cudaMemcpyHostToDevice, st));
    LL_CUDA(cudaMemcpyAsync(m->btok + seq, &m->btok_host[seq], sizeof(int), cudaMemcpyHostToDevice, st));
    LL_CUDA(cudaStreamSynchronize(st));
    if (first_token_out) {
        *first_token_out = first;
    }
    return QMM_OK;
}

int qmm_llama_batch_decode_enqueue(qmm_llama* m, int steps, void* stream)
{
    if (!m || m->batch == 0) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_decode: no batch (qmm_llama_batch_create first)");
    }
    int deepest = 0;
    for (int p : m->bpos_host) {
        deepest = std::max(deepest, p);
    }
    if (steps < 1 || m->bsteps_host + steps > m->batch_max_steps || deepest + m->bsteps_host + steps > m->cfg.max_seq) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_decode: step count outside the batch's capacity");
    }
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!m->bgraph) {
        if (st == nullptr) {
            return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_decode needs a non-default stream (graph capture)");
        }
        LL_QMM(enqueue_batch_step(m, st));  // eager once: one-time kernel set-up happens outside a capture
        m->bsteps_host += 1;
        steps -= 1;
        cudaGraph_t g = nullptr;
        LL_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_batch_step(m, st);
        const cudaError_t e = cudaStreamEndCapture(st, &g);
        if (rc != QMM_OK) {
            if (g) {
                cudaGraphDestroy(g);
            }
            return rc;
        }
        LL_CUDA(e);
        LL_CUDA(cudaGraphInstantiate(&m->bgraph, g, 0));
        cudaGraphDestroy(g);
    }
    for (int s = 0; s < steps; ++s) {
        LL_CUDA(cudaGraphLaunch(m->bgraph, st));
    }
    m->bsteps_host += steps;
    return QMM_OK;
}

int qmm_llama_batch_generated_tokens(qmm_llama* m, int first_step, int steps, int32_t* tokens_out_host, void* stream)
{
    if (!m || m->batch == 0 || !tokens_out_host || first_step < 0 || steps < 0 || first_step + steps > m->bsteps_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_generated_tokens: range outside the steps taken so far");
    }
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_QMM(read_back(m, tokens_out_host, m->bout + (size_t)first_step * m->batch,
                     (size_t)steps * m->batch * sizeof(int), st));
    return check_status(m);
}

int qmm_llama_batch_decode(qmm_llama* m, int steps, int32_t* tokens_out_host, void* stream)
{
    if (!tokens_out_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_batch_decode: output pointer is null");
    }
    const int first = m ? m->bsteps_host : 0;
    LL_QMM(qmm_llama_batch_decode_enqueue(m, steps, stream));
    return qmm_llama_batch_generated_tokens(m, first, steps, tokens_out_host, stream);
}

int qmm_llama_last_logits(qmm_llama* m, float* logits_host, void* stream)
{
    if (!m || !logits_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_last_logits: null argument");
    }
    LL_GUARD(m);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_CUDA(cudaMemcpyAsync(logits_host, m->logits, (size_t)m->vl * sizeof(float), cudaMemcpyDeviceToHost, st));
    LL_CUDA(cudaStreamSynchronize(st));
    return QMM_OK;
}

}  // extern "C"

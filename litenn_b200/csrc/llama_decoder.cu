// LLaMA decoder harness (include/litenn_llama.h): buffers, KV cache, the per-token launch
// sequence captured into a CUDA graph (or the persistent kernel of llama_mega.cu), the prefill
// sequence, and the tensor-parallel mode: NCCL all-reduces in prefill, and in decode either
// NCCL or the peer-memory exchange built into the matvec and norm kernels.  The linears are the
// quantized kernels of qmm_gemv.cu / qmm_gemm.cu, called through the library's own C ABI.
#include "../../include/litenn_llama.h"

#include <dlfcn.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "llama_kernels.h"
#include "qmm_common.cuh"

int qmm_internal_fail(int code, const char* message);
int qmm_internal_weight_view(const qmm_weight* w, qmm::WeightView* out);
int qmm_internal_gemv_packed(const qmm_weight* w, const void* packed_dev, float* y_dev, int m,
                             const qmm::PeerScatter* scatter, void* stream);

using namespace qmm;

namespace {

// ---- NCCL, resolved at run time ----------------------------------------------------------------
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, /* ncclUniqueId by value: 128 bytes */ struct Id128, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
};
struct Id128 {
    char bytes[128];
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
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
    g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
    g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(dlsym(lib, "ncclAllReduce"));
    g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(dlsym(lib, "ncclAllGather"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.AllGather) {
        dlclose(lib);
        return qmm_internal_fail(QMM_E_UNSUPPORTED, "the NCCL library lacks a required symbol");
    }
    g_nccl.lib = lib;
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
    float* final_norm = nullptr;
    uint8_t* embd = nullptr;
    std::vector<void*> allocs;
    // decode buffers
    float *h = nullptr, *h2 = nullptr, *y = nullptr, *y2 = nullptr, *qkv = nullptr, *gu = nullptr, *logits = nullptr;
    uint8_t *pk_d = nullptr, *pk_ctx = nullptr, *pk_ffn = nullptr;
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
    // direct peer exchange of the two per-block sums (replaces the NCCL all-reduce in decode)
    uint2* xchg = nullptr;       // [2][tp][d_model] packets {value, exchange number}, exported over CUDA IPC
    uint2* peer_xchg[8] = {};    // the same buffer of every peer, mapped here
    bool xchg_ready = false;
    // persistent-kernel decode path
    int decode_mode = QMM_LL_DECODE_AUTO;
    int mega_state = 0;  // 0 = not examined, 1 = ready, -1 = unavailable for this model
    std::string mega_why;
    MegaArgs mega = {};
    int mega_grid = 0;
    int* mega_status = nullptr;
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

// logits -> (value, index) of this rank -> winner over ranks -> token, position, output list
int pick_token(qmm_llama* m, cudaStream_t st)
{
    const qmm_llama_config& c = m->cfg;
    LL_CUDA(ll_argmax(m->logits, m->vl, m->vl * c.tp_rank, ARGMAX_CTAS, m->pair, st));
    const int* pairs = m->pair;
    if (c.tp_size > 1) {
        if (g_nccl.AllGather(m->pair, m->pairs, 2 * ARGMAX_CTAS, NCCL_INT32, m->comm, st) != 0) {
            return qmm_internal_fail(QMM_E_CUDA, "ncclAllGather failed");
        }
        pairs = m->pairs;
    }
    LL_CUDA(ll_commit_token(pairs, c.tp_size * ARGMAX_CTAS, m->token, m->pos, m->out_tokens, m->out_count, st));
    return QMM_OK;
}

// Exchange `site` (0 .. 2*n_layers-1) of a token alternates between two receive buffers: a
// rank can only be one exchange ahead of a peer (it needs the peer's addend to finish its own
// sum), so the buffer it overwrites has been read.
PeerScatter scatter_for(const qmm_llama* m, int site)
{
    PeerScatter ps = {};
    if (!m->xchg_ready) {
        return ps;
    }
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
    return ps;
}

PeerGather gather_for(const qmm_llama* m, int site)
{
    PeerGather pg = {};
    if (!m->xchg_ready || site < 0) {
        return pg;
    }
    const qmm_llama_config& c = m->cfg;
    pg.recv = m->xchg + (size_t)(site & 1) * c.tp_size * c.d_model;
    pg.tp_rank = c.tp_rank;
    pg.tp_size = c.tp_size;
    pg.pos = m->pos;
    pg.sites = 2 * c.n_layers;
    pg.site = site;
    pg.status = m->mega_status;
    return pg;
}

// K-split matvec whose result is summed over the ranks: peer scatter when the exchange
// buffers are mapped, else an NCCL all-reduce.
int linear_sum(qmm_llama* m, const qmm_weight* w, const uint8_t* packed, float* y, int site, cudaStream_t st)
{
    if (m->xchg_ready) {
        const PeerScatter ps = scatter_for(m, site);
        return qmm_internal_gemv_packed(w, packed, y, 1, &ps, st);
    }
    LL_QMM(qmm_gemv_packed(w, packed, y, 1, st));
    return all_reduce(m, y, m->cfg.d_model, st);
}

// `site` >= 0: `add` is this rank's addend of exchange `site` (decode with mapped peers).
int final_head(qmm_llama* m, const float* h, const float* add, int site, cudaStream_t st)
{
    const qmm_llama_config& c = m->cfg;
    LL_CUDA(ll_resid_rmsnorm_pack(h, add, m->final_norm, c.rms_eps, c.d_model, m->pk_d, nullptr, gather_for(m, site), st));
    LL_QMM(qmm_gemv_packed(m->head, m->pk_d, m->logits, 1, st));
    return pick_token(m, st);
}

// One token at position *pos: everything reads its inputs from device memory, so the same
// sequence can be replayed from a CUDA graph.
int enqueue_decode_step(qmm_llama* m, cudaStream_t st)
{
    const qmm_llama_config& c = m->cfg;
    // The residual stream alternates between two buffers: the norm kernel reads one and writes
    // the other, so its CTAs never race on it.
    float* ha = m->h;
    float* hb = m->h2;
    LL_CUDA(ll_embed_rows(c.embd_fmt, m->embd, m->token, 1, c.d_model, ha, st));
    for (int l = 0; l < c.n_layers; ++l) {
        Layer& L = m->layers[l];
        LL_CUDA(ll_resid_rmsnorm_pack(ha, l == 0 ? nullptr : m->y2, L.attn_norm, c.rms_eps, c.d_model, m->pk_d, hb,
                                      gather_for(m, l == 0 ? -1 : 2 * l - 1), st));
        LL_QMM(qmm_gemv_packed(L.w[QMM_LL_QKV], m->pk_d, m->qkv, 1, st));
        LL_CUDA(ll_attn_fused(m->qkv, m->pos, m->hl, m->kvl, c.head_dim, c.rope_dim, m->rope_cos, m->rope_sin,
                              c.max_seq, L.cache_k, L.cache_v, m->pk_ctx, st));
        LL_QMM(linear_sum(m, L.w[QMM_LL_O], m->pk_ctx, m->y, 2 * l, st));
        LL_CUDA(ll_resid_rmsnorm_pack(hb, m->y, L.ffn_norm, c.rms_eps, c.d_model, m->pk_d, ha, gather_for(m, 2 * l), st));
        LL_QMM(qmm_gemv_packed(L.w[QMM_LL_GU], m->pk_d, m->gu, 1, st));
        LL_CUDA(ll_silu_mul_pack(m->gu, m->ffl, m->pk_ffn, st));
        LL_QMM(linear_sum(m, L.w[QMM_LL_DOWN], m->pk_ffn, m->y2, 2 * l + 1, st));
    }
    return final_head(m, ha, m->y2, 2 * c.n_layers - 1, st);
}

// Sets up the persistent-kernel path if this model fits it; otherwise records why not.
int prepare_mega(qmm_llama* m)
{
    if (m->mega_state != 0) {
        return QMM_OK;
    }
    m->mega_state = -1;
    const qmm_llama_config& c = m->cfg;
    if (c.tp_size != 1) {
        m->mega_why = "tensor-parallel models use the per-operator path";
        return QMM_OK;
    }
    int sms = 0, coop = 0;
    LL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, m->device));
    LL_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, m->device));
    if (!coop || sms < 1) {
        m->mega_why = "the device does not support cooperative launches";
        return QMM_OK;
    }
    const int L = c.n_layers, grid = sms;
    std::vector<MegaLinear> lin((size_t)4 * L + 1);
    std::vector<MegaLayer> layers((size_t)L);
    int kc_max = 1;
    auto fill = [&](MegaLinear& d, const qmm_weight* w, float* y) -> int {
        WeightView v;
        LL_QMM(qmm_internal_weight_view(w, &v));
        d.tiles = v.tiles;
        d.y = y;
        d.n = (int)v.n;
        d.rt = v.rt;
        d.kc = v.kc;
        d.fmt = v.fmt;
        d.tile_bytes = (uint32_t)tile_bytes(v.fmt);
        d.wpr = ll_mega_pick_wpr(v.rt, v.kc, grid);
        kc_max = v.kc > kc_max ? v.kc : kc_max;
        return QMM_OK;
    };
    for (int l = 0; l < L; ++l) {
        Layer& ly = m->layers[l];
        LL_QMM(fill(lin[4 * l + 0], ly.w[QMM_LL_QKV], m->qkv));
        LL_QMM(fill(lin[4 * l + 1], ly.w[QMM_LL_O], m->y));
        LL_QMM(fill(lin[4 * l + 2], ly.w[QMM_LL_GU], m->gu));
        LL_QMM(fill(lin[4 * l + 3], ly.w[QMM_LL_DOWN], m->y2));
        layers[l].attn_norm = ly.attn_norm;
        layers[l].ffn_norm = ly.ffn_norm;
        layers[l].cache_k = ly.cache_k;
        layers[l].cache_v = ly.cache_v;
    }
    LL_QMM(fill(lin[4 * L], m->head, m->logits));
    for (const MegaLinear& d : lin) {
        if (d.tile_bytes > (uint32_t)MEGA_RING_BYTES) {
            m->mega_why = "a weight tile does not fit the per-warp ring";
            return QMM_OK;
        }
    }
    if (c.d_model > 2 * 256 * MEGA_WARPS || ll_mega_smem_bytes(c.d_model, c.head_dim, kc_max, c.n_layers) > 227 * 1024) {
        m->mega_why = "the model's activations do not fit one CTA's shared memory";
        return QMM_OK;
    }
    MegaArgs& a = m->mega;
    MegaLinear* lin_dev = nullptr;
    MegaLayer* layers_dev = nullptr;
    unsigned int* sync = nullptr;
    a.nsplit = grid / m->hl > 0 ? grid / m->hl : 1;
    LL_QMM(dev_alloc(m, &lin_dev, lin.size()));
    LL_QMM(dev_alloc(m, &layers_dev, layers.size()));
    LL_QMM(dev_alloc(m, &a.part, (size_t)m->hl * a.nsplit * (c.head_dim + 4)));
    LL_QMM(dev_alloc(m, &a.cand, (size_t)2 * grid));
    LL_QMM(dev_alloc(m, &sync, 2));
    LL_CUDA(cudaMemcpy(lin_dev, lin.data(), lin.size() * sizeof(MegaLinear), cudaMemcpyHostToDevice));
    LL_CUDA(cudaMemcpy(layers_dev, layers.data(), layers.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice));
    a.lin = lin_dev;
    a.layers = layers_dev;
    a.final_norm = m->final_norm;
    a.embd = m->embd;
    a.embd_fmt = c.embd_fmt;
    a.n_layers = L;
    a.d_model = c.d_model;
    a.n_heads = m->hl;
    a.n_kv = m->kvl;
    a.hd = c.head_dim;
    a.rope_dim = c.rope_dim;
    a.ffn = m->ffl;
    a.vocab = m->vl;
    a.max_seq = c.max_seq;
    a.eps = c.rms_eps;
    a.rope_cos = m->rope_cos;
    a.rope_sin = m->rope_sin;
    a.token = m->token;
    a.pos = m->pos;
    a.out_tokens = m->out_tokens;
    a.out_count = m->out_count;
    a.sync = sync;
    a.status = m->mega_status;
    a.kc_max = kc_max;
    m->mega_grid = grid;
    m->mega_state = 1;
    return QMM_OK;
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
        if (!L.attn_norm || !L.ffn_norm) {
            return qmm_internal_fail(QMM_E_INVALID, "a layer norm has not been set");
        }
    }
    if (!m->head || !m->final_norm || !m->embd) {
        return qmm_internal_fail(QMM_E_INVALID, "output weight, final norm or embedding has not been set");
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
    LL_CUDA(cudaMemsetAsync(m->xchg, 0, (size_t)2 * m->cfg.tp_size * m->cfg.d_model * sizeof(uint2), st));
    return all_reduce(m, m->y, 1, st);
}

// After a synchronize: did the persistent kernel give up on a bounded wait?
int check_mega_status(qmm_llama* m)
{
    if (m->mega_state != 1 && !m->xchg_ready) {
        return QMM_OK;
    }
    int word = 0;
    LL_CUDA(cudaMemcpy(&word, m->mega_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (word != 0) {
        char buf[128];
        snprintf(buf, sizeof buf, "decode: a bounded wait ran out (status %d: 1 weight copy, 3 grid barrier, 5 peer addend)",
                 word);
        return qmm_internal_fail(QMM_E_KERNEL, buf);
    }
    return QMM_OK;
}

}  // namespace

extern "C" {

int qmm_llama_set_decode_mode(qmm_llama* m, int mode)
{
    if (!m || mode < QMM_LL_DECODE_AUTO || mode > QMM_LL_DECODE_PERSISTENT) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_set_decode_mode: invalid argument");
    }
    m->decode_mode = mode;
    return QMM_OK;
}

int qmm_llama_create(int device, const qmm_llama_config* cfg, qmm_llama** out)
{
    if (!cfg || !out) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_create: null argument");
    }
    *out = nullptr;
    const qmm_llama_config& c = *cfg;
    if (c.n_layers < 1 || c.d_model < 1 || c.n_heads < 1 || c.n_kv_heads < 1 || (c.head_dim != 64 && c.head_dim != 128) ||
        c.rope_dim > c.head_dim || (c.rope_dim % 2) != 0 || c.tp_size < 1 ||
        c.tp_rank < 0 || c.tp_rank >= c.tp_size || c.max_seq < 1 || c.vocab < 1 || c.ffn < 1) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_create: invalid hyperparameters");
    }
    if (c.n_heads % c.n_kv_heads != 0 || c.n_heads % c.tp_size != 0 || c.n_kv_heads % c.tp_size != 0 ||
        c.ffn % c.tp_size != 0 || c.vocab % c.tp_size != 0) {
        return qmm_internal_fail(QMM_E_INVALID,
                                 "heads, kv heads, ffn width and vocabulary must divide over the tensor-parallel ranks");
    }
    if (block_elems(c.embd_fmt) == 0 || c.d_model % block_elems(c.embd_fmt) != 0) {
        return qmm_internal_fail(QMM_E_INVALID, "embedding format or width not supported");
    }
    LL_CUDA(cudaSetDevice(device));
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
#define LL_TRY(x)                \
    if (rc == QMM_OK) {          \
        rc = (x);                \
    }
    LL_TRY(dev_alloc(m, &m->h, d));
    LL_TRY(dev_alloc(m, &m->mega_status, 1));
    LL_TRY(dev_alloc(m, &m->h2, d));
    LL_TRY(dev_alloc(m, &m->y, d));
    LL_TRY(dev_alloc(m, &m->y2, d));
    LL_TRY(dev_alloc(m, &m->qkv, qkv_w));
    LL_TRY(dev_alloc(m, &m->gu, (size_t)2 * m->ffl));
    LL_TRY(dev_alloc(m, &m->logits, m->vl));
    LL_TRY(qmm_packed_activation_bytes(d, 1, &pk));
    LL_TRY(dev_alloc(m, &m->pk_d, pk));
    LL_TRY(qmm_packed_activation_bytes((int64_t)m->hl * hd, 1, &pk));
    LL_TRY(dev_alloc(m, &m->pk_ctx, pk));
    LL_TRY(qmm_packed_activation_bytes(m->ffl, 1, &pk));
    LL_TRY(dev_alloc(m, &m->pk_ffn, pk));
    LL_TRY(dev_alloc(m, &m->rope_cos, (size_t)c.max_seq * (c.rope_dim / 2)));
    LL_TRY(dev_alloc(m, &m->rope_sin, (size_t)c.max_seq * (c.rope_dim / 2)));
    LL_TRY(dev_alloc(m, &m->pos, 1));
    LL_TRY(dev_alloc(m, &m->token, 1));
    LL_TRY(dev_alloc(m, &m->out_tokens, (size_t)c.max_seq + 8));
    LL_TRY(dev_alloc(m, &m->out_count, 1));
    LL_TRY(dev_alloc(m, &m->pair, 2 * ARGMAX_CTAS));
    LL_TRY(dev_alloc(m, &m->pairs, (size_t)2 * ARGMAX_CTAS * c.tp_size));
    LL_TRY(dev_alloc(m, &m->final_norm, d));
    for (int l = 0; l < c.n_layers && rc == QMM_OK; ++l) {
        LL_TRY(dev_alloc(m, &m->layers[l].attn_norm, d));
        LL_TRY(dev_alloc(m, &m->layers[l].ffn_norm, d));
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
    cudaSetDevice(m->device);
    if (m->graph) {
        cudaGraphExecDestroy(m->graph);
    }
    if (m->comm && g_nccl.CommDestroy) {
        g_nccl.CommDestroy(m->comm);
    }
    for (uint2* p : m->peer_xchg) {
        if (p) {
            cudaIpcCloseMemHandle(p);
        }
    }
    for (void* p : m->allocs) {
        cudaFree(p);
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
    LL_CUDA(cudaSetDevice(m->device));
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
    LL_CUDA(cudaSetDevice(m->device));
    LL_QMM(dev_alloc(m, &m->embd, payload_bytes));
    LL_CUDA(cudaMemcpy(m->embd, payload_host, payload_bytes, cudaMemcpyHostToDevice));
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
    LL_CUDA(cudaSetDevice(m->device));
    Id128 uid;
    memcpy(uid.bytes, id, 128);
    if (g_nccl.CommInitRank(&m->comm, m->cfg.tp_size, uid, m->cfg.tp_rank) != 0) {
        return qmm_internal_fail(QMM_E_CUDA, "ncclCommInitRank failed");
    }
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
    LL_CUDA(cudaSetDevice(m->device));
    if (!m->xchg) {
        LL_QMM(dev_alloc(m, &m->xchg, (size_t)2 * m->cfg.tp_size * m->cfg.d_model));
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
    if (c.tp_size > 8) {
        return qmm_internal_fail(QMM_E_UNSUPPORTED, "the peer exchange serves up to 8 ranks");
    }
    LL_CUDA(cudaSetDevice(m->device));
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
    if (m->graph) {  // a graph captured earlier still holds the all-reduce form
        cudaGraphExecDestroy(m->graph);
        m->graph = nullptr;
    }
    return rearm_exchange(m, static_cast<cudaStream_t>(stream));
}

int qmm_llama_reset(qmm_llama* m, void* stream)
{
    if (!m) {
        return qmm_internal_fail(QMM_E_INVALID, "model handle is null");
    }
    LL_CUDA(cudaSetDevice(m->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_CUDA(cudaMemsetAsync(m->pos, 0, sizeof(int), st));
    LL_CUDA(cudaMemsetAsync(m->out_count, 0, sizeof(int), st));
    LL_QMM(rearm_exchange(m, st));
    LL_CUDA(cudaStreamSynchronize(st));
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
    LL_CUDA(cudaSetDevice(m->device));
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
    LL_QMM(final_head(m, m->hr + (size_t)(n - 1) * d, m->y2r + (size_t)(n - 1) * d, -1, st));
    int32_t tok = 0;
    LL_CUDA(cudaMemcpyAsync(&tok, m->token, sizeof(int), cudaMemcpyDeviceToHost, st));
    LL_CUDA(cudaStreamSynchronize(st));
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
    LL_CUDA(cudaSetDevice(m->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (m->decode_mode == QMM_LL_DECODE_PERSISTENT) {
        LL_QMM(prepare_mega(m));
        if (m->mega_state == 1) {
            for (int s = 0; s < steps; ++s) {
                LL_CUDA(ll_mega_decode(m->mega, m->mega_grid, st));
            }
            m->host_pos += steps;
            m->host_count += steps;
            return QMM_OK;
        }
        return qmm_internal_fail(QMM_E_UNSUPPORTED, ("persistent decode kernel unavailable: " + m->mega_why).c_str());
    }
    if (!m->graph) {
        if (st == nullptr) {
            return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_decode needs a non-default stream (graph capture)");
        }
        // The first token runs eagerly (it also performs every kernel's one-time set-up outside
        // a capture); the same sequence is then captured once and replayed for all later tokens.
        LL_QMM(enqueue_decode_step(m, st));
        m->host_pos += 1;
        m->host_count += 1;
        steps -= 1;
        if (steps == 0) {
            return QMM_OK;
        }
        cudaGraph_t g = nullptr;
        LL_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_decode_step(m, st);
        cudaError_t e = cudaStreamEndCapture(st, &g);
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
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_CUDA(cudaMemcpyAsync(tokens_out_host, m->out_tokens + first, (size_t)steps * sizeof(int), cudaMemcpyDeviceToHost,
                            st));
    LL_CUDA(cudaStreamSynchronize(st));
    return check_mega_status(m);
}

int qmm_llama_step_host(qmm_llama* m, int32_t token_in, int32_t* token_out, void* stream)
{
    if (!m || !token_out) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_step_host: null argument");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_CUDA(cudaSetDevice(m->device));
    LL_CUDA(cudaMemcpyAsync(m->token, &token_in, sizeof(int), cudaMemcpyHostToDevice, st));
    LL_QMM(qmm_llama_decode_enqueue(m, 1, stream));
    LL_CUDA(cudaMemcpyAsync(token_out, m->token, sizeof(int), cudaMemcpyDeviceToHost, st));
    LL_CUDA(cudaStreamSynchronize(st));
    return check_mega_status(m);
}

int qmm_llama_last_logits(qmm_llama* m, float* logits_host, void* stream)
{
    if (!m || !logits_host) {
        return qmm_internal_fail(QMM_E_INVALID, "qmm_llama_last_logits: null argument");
    }
    LL_CUDA(cudaSetDevice(m->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LL_CUDA(cudaMemcpyAsync(logits_host, m->logits, (size_t)m->vl * sizeof(float), cudaMemcpyDeviceToHost, st));
    LL_CUDA(cudaStreamSynchronize(st));
    return QMM_OK;
}

}  // extern "C"

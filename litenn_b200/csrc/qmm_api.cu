// C ABI of the library (include/litenn_qmm.h): argument validation, device
// memory ownership, per-(device,stream) scratch, and dispatch to the kernels.
#include "../../include/litenn_qmm.h"

#include <cstdarg>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <utility>

#include "qmm_internal.h"
#include "qmm_kernels.h"

using namespace qmm;

struct qmm_weight {
    int fmt;
    int device;
    int sm_count;
    int64_t n, k;
    int rt, kc;
    int64_t payload_bytes;
    size_t packed_bytes;
    uint8_t* base;  // [rt][kc] packed tiles
};

namespace {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int fail_cuda(cudaError_t e, const char* what)
{
    return fail(QMM_E_CUDA, "%s failed: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

#define QMM_CUDA(call)                         \
    do {                                       \
        cudaError_t e_ = (call);               \
        if (e_ != cudaSuccess) {               \
            return fail_cuda(e_, #call);       \
        }                                      \
    } while (0)

bool supported_format(int fmt)
{
    return fmt == FMT_Q4_0 || fmt == FMT_Q8_0 || fmt == FMT_Q4_K || fmt == FMT_Q6_K;
}

// Formats qmm_dequantize_raw and qmm_block_layout also know: carried as payloads, never multiplied.
bool dequant_only_format(int fmt)
{
    return fmt == FMT_Q4_1 || fmt == FMT_Q5_0 || fmt == FMT_Q5_1 || fmt == FMT_Q2_K || fmt == FMT_Q3_K || fmt == FMT_Q5_K;
}

size_t align_up(size_t v, size_t a)
{
    return (v + a - 1) / a * a;
}

WeightView view_of(const qmm_weight* w)
{
    WeightView v;
    v.tiles = w->base;
    v.n = w->n;
    v.k = w->k;
    v.rt = w->rt;
    v.kc = w->kc;
    v.fmt = w->fmt;
    return v;
}

// Scratch for the packed activations, one per (device, stream); grown on demand.
struct Workspace {
    uint8_t* base = nullptr;
    size_t bytes = 0;
    int flip = 0;
    void* conv = nullptr;      // bf16 copy of fp32 activations (qmm_gemm_f32)
    size_t conv_bytes = 0;
    float* stage_x = nullptr;  // device staging for the host-buffer entry point
    float* stage_y = nullptr;
    size_t stage_x_bytes = 0;
    size_t stage_y_bytes = 0;
};

std::mutex g_ws_mutex;
std::map<std::pair<int, void*>, Workspace> g_workspaces;
// One int per device that kernels set non-zero when a bounded wait runs out.
std::map<int, int*> g_status_words;

int get_status_word(int device, int** out)
{
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    auto it = g_status_words.find(device);
    if (it == g_status_words.end()) {
        int* p = nullptr;
        QMM_CUDA(cudaMalloc(&p, sizeof(int)));
        QMM_CUDA(cudaMemset(p, 0, sizeof(int)));
        it = g_status_words.emplace(device, p).first;
    }
    *out = it->second;
    return QMM_OK;
}

// Two activation buffers of `one` bytes per (device, stream), handed out alternately.
int get_workspace_half(int device, void* stream, size_t one, uint8_t** out)
{
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    Workspace& ws = g_workspaces[std::make_pair(device, stream)];
    const size_t bytes = 2 * one;
    if (ws.bytes < bytes) {
        if (ws.base) {
            // the old buffer may still be read by work queued on the stream
            QMM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
            QMM_CUDA(cudaFree(ws.base));
            ws.base = nullptr;
            ws.bytes = 0;
        }
        const size_t want = align_up(bytes, 1 << 20);
        QMM_CUDA(cudaMalloc(&ws.base, want));
        ws.bytes = want;
    }
    *out = ws.base + (ws.flip ? ws.bytes / 2 : 0);
    ws.flip ^= 1;
    return QMM_OK;
}

int create_impl(int device, int fmt, const void* payload, size_t payload_bytes, int payload_on_device, int64_t n,
                int64_t k, int split, int tp_rank, int tp_size, void* stream_v, qmm_weight** out)
{
    if (!out) {
        return fail(QMM_E_INVALID, "qmm_weight_create: out is null");
    }
    *out = nullptr;
    if (!supported_format(fmt)) {
        return fail(QMM_E_UNSUPPORTED, "block format %d is not one of Q4_0(1), Q8_0(5), Q4_K(9), Q6_K(11)", fmt);
    }
    if (!payload) {
        return fail(QMM_E_INVALID, "payload is null");
    }
    if (n <= 0 || k <= 0) {
        return fail(QMM_E_INVALID, "invalid expressed shape [%lld, %lld]", (long long)n, (long long)k);
    }
    const int elems = block_elems(fmt);
    const int bbytes = block_bytes(fmt);
    if (k % elems != 0) {
        return fail(QMM_E_INVALID, "row width %lld is incompatible with ggml block size %d", (long long)k, elems);
    }
    const int64_t row_bytes = (k / elems) * bbytes;
    if ((int64_t)payload_bytes != n * row_bytes) {
        return fail(QMM_E_INVALID, "payload byte count %zu does not match expressed shape %lldx%lld (%lld bytes)",
                    payload_bytes, (long long)n, (long long)k, (long long)(n * row_bytes));
    }
    int64_t row0 = 0, blk0 = 0, n_loc = n, k_loc = k;
    if (split != QMM_SPLIT_NONE) {
        if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) {
            return fail(QMM_E_INVALID, "invalid shard %d of %d", tp_rank, tp_size);
        }
        if (split == QMM_SPLIT_N) {
            if (n % tp_size != 0) {
                return fail(QMM_E_INVALID, "%lld rows do not divide over %d ranks", (long long)n, tp_size);
            }
            n_loc = n / tp_size;
            row0 = n_loc * tp_rank;
        } else if (split == QMM_SPLIT_K) {
            if (k % tp_size != 0 || (k / tp_size) % elems != 0) {
                return fail(QMM_E_INVALID,
                            "row width %lld cannot be cut into %d shards of whole %d-element blocks", (long long)k,
                            tp_size, elems);
            }
            k_loc = k / tp_size;
            blk0 = (k_loc / elems) * tp_rank;
        } else {
            return fail(QMM_E_INVALID, "unknown split kind %d", split);
        }
    }
    int count = 0;
    QMM_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) {
        return fail(QMM_E_INVALID, "device index %d out of range (%d devices)", device, count);
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    int sm_count = 0;
    QMM_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    qmm_weight* w = new (std::nothrow) qmm_weight();
    if (!w) {
        return fail(QMM_E_INVALID, "out of host memory");
    }
    w->sm_count = sm_count;
    w->fmt = fmt;
    w->device = device;
    w->n = n_loc;
    w->k = k_loc;
    w->rt = (int)((n_loc + TILE_ROWS - 1) / TILE_ROWS);
    w->kc = (int)((k_loc + TILE_K - 1) / TILE_K);
    w->payload_bytes = n_loc * (k_loc / elems) * bbytes;
    const size_t tiles = (size_t)w->rt * w->kc;
    w->packed_bytes = align_up(tiles * tile_bytes(fmt), 256);
    cudaError_t e = cudaMalloc(&w->base, w->packed_bytes);
    if (e != cudaSuccess) {
        delete w;
        return fail_cuda(e, "cudaMalloc(packed weight)");
    }

    // Stage only the byte range of the raw payload this shard reads.
    const uint8_t* raw_dev = nullptr;
    uint8_t* staged = nullptr;
    const int64_t first_byte = row0 * row_bytes;
    const int64_t span_bytes = n_loc * row_bytes;
    if (payload_on_device) {
        raw_dev = static_cast<const uint8_t*>(payload);
    } else {
        e = cudaMalloc(&staged, (size_t)span_bytes);
        if (e == cudaSuccess) {
            e = cudaMemcpyAsync(staged, static_cast<const uint8_t*>(payload) + first_byte, (size_t)span_bytes,
                                cudaMemcpyHostToDevice, stream);
        }
        if (e != cudaSuccess) {
            if (staged) {
                cudaFree(staged);
            }
            cudaFree(w->base);
            delete w;
            return fail_cuda(e, "staging the raw payload");
        }
        raw_dev = staged;  // holds rows row0.. only
        row0 = 0;
    }
    RawSource src;
    src.base = raw_dev;
    src.row_bytes = row_bytes;
    src.row0 = row0;
    src.blk0 = blk0;
    src.n = n_loc;
    src.nblk = k_loc / elems;
    e = launch_repack(fmt, src, w->rt, w->kc, w->base, w->sm_count, stream);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(stream);
    }
    if (staged) {
        cudaFree(staged);
    }
    if (e != cudaSuccess) {
        cudaFree(w->base);
        delete w;
        return fail_cuda(e, "repack");
    }
    *out = w;
    return QMM_OK;
}

int check_weight(const qmm_weight* w, const char* who)
{
    if (!w) {
        return fail(QMM_E_INVALID, "%s: weight handle is null", who);
    }
    return QMM_OK;
}

}  // namespace

// Error reporting for the other translation units of the library (llama_decoder.cu).
int qmm_internal_fail(int code, const char* message)
{
    return fail(code, "%s", message);
}

// For the decoder (llama_decoder.cu): the device-side view of a packed weight.
int qmm_internal_weight_view(const qmm_weight* w, qmm::WeightView* out)
{
    if (!w || !out) {
        return qmm_internal_fail(QMM_E_INVALID, "weight handle is null");
    }
    *out = view_of(w);
    return QMM_OK;
}

extern "C" {

int qmm_abi_version(void)
{
    return QMM_ABI_VERSION;
}

const char* qmm_last_error(void)
{
    return g_last_error.c_str();
}

int qmm_block_layout(int fmt, int* elems_per_block, int* bytes_per_block)
{
    if (!supported_format(fmt) && !dequant_only_format(fmt)) {
        return fail(QMM_E_UNSUPPORTED, "block format %d is not supported", fmt);
    }
    if (elems_per_block) {
        *elems_per_block = block_elems(fmt);
    }
    if (bytes_per_block) {
        *bytes_per_block = block_bytes(fmt);
    }
    return QMM_OK;
}

int qmm_device_count(void)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return count;
}

int qmm_weight_create(int device, int fmt, const void* payload, size_t payload_bytes, int payload_on_device,
                      int64_t n, int64_t k, void* stream, qmm_weight** out)
{
    return create_impl(device, fmt, payload, payload_bytes, payload_on_device, n, k, QMM_SPLIT_NONE, 0, 1, stream,
                       out);
}

int qmm_weight_create_shard(int device, int fmt, const void* payload, size_t payload_bytes, int payload_on_device,
                            int64_t n, int64_t k, int split, int tp_rank, int tp_size, void* stream,
                            qmm_weight** out)
{
    return create_impl(device, fmt, payload, payload_bytes, payload_on_device, n, k, split, tp_rank, tp_size,
                       stream, out);
}

int qmm_weight_destroy(qmm_weight* w)
{
    if (!w) {
        return QMM_OK;
    }
    DeviceGuard guard(w->device);
    cudaError_t e = cudaFree(w->base);
    delete w;
    if (e != cudaSuccess) {
        return fail_cuda(e, "cudaFree(packed weight)");
    }
    return QMM_OK;
}

int qmm_weight_get_info(const qmm_weight* w, qmm_weight_info* info)
{
    if (int rc = check_weight(w, "qmm_weight_get_info")) {
        return rc;
    }
    if (!info) {
        return fail(QMM_E_INVALID, "info is null");
    }
    info->fmt = w->fmt;
    info->device = w->device;
    info->n = w->n;
    info->k = w->k;
    info->payload_bytes = w->payload_bytes;
    info->packed_bytes = (int64_t)w->packed_bytes;
    return QMM_OK;
}

int qmm_dequantize(const qmm_weight* w, float* out_dev, void* stream)
{
    if (int rc = check_weight(w, "qmm_dequantize")) {
        return rc;
    }
    if (!out_dev) {
        return fail(QMM_E_INVALID, "output pointer is null");
    }
    DeviceGuard guard(w->device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    QMM_CUDA(launch_dequant_packed(view_of(w), out_dev, w->sm_count, static_cast<cudaStream_t>(stream)));
    return QMM_OK;
}

int qmm_dequantize_raw(int device, int fmt, const void* payload_dev, int64_t n, int64_t k, float* out_dev,
                       void* stream)
{
    if (!supported_format(fmt) && !dequant_only_format(fmt)) {
        return fail(QMM_E_UNSUPPORTED, "block format %d is not supported", fmt);
    }
    if (!payload_dev || !out_dev || n <= 0 || k <= 0 || k % block_elems(fmt) != 0) {
        return fail(QMM_E_INVALID, "invalid arguments to qmm_dequantize_raw");
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    int sm_count = 0;
    QMM_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    QMM_CUDA(launch_dequant_raw(fmt, static_cast<const uint8_t*>(payload_dev), n, k, out_dev, sm_count,
                                static_cast<cudaStream_t>(stream)));
    return QMM_OK;
}

int qmm_packed_activation_bytes(int64_t k, int m, size_t* bytes)
{
    if (!bytes || k <= 0 || m < 1 || m > QMM_GEMV_MAX_BATCH) {
        return fail(QMM_E_INVALID, "qmm_packed_activation_bytes: invalid k=%lld m=%d", (long long)k, m);
    }
    const int kc = (int)((k + TILE_K - 1) / TILE_K);
    *bytes = align_up(m == 1 ? xpack1_bytes(kc) : xpack_bytes(kc, xpack_ncp(m)), 256);
    return QMM_OK;
}

int qmm_pack_activations(int device, const float* x_dev, int m, int64_t k, void* packed_dev, void* stream_v)
{
    if (!x_dev || !packed_dev) {
        return fail(QMM_E_INVALID, "qmm_pack_activations: null pointer");
    }
    if (m < 1 || m > QMM_GEMV_MAX_BATCH || k <= 0 || k % 32 != 0) {
        return fail(QMM_E_INVALID, "qmm_pack_activations: batch %d outside 1..%d or k=%lld not a multiple of 32", m,
                    QMM_GEMV_MAX_BATCH, (long long)k);
    }
    if ((reinterpret_cast<uintptr_t>(packed_dev) & 15u) != 0) {
        return fail(QMM_E_INVALID, "qmm_pack_activations: packed buffer must be 16-byte aligned");
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    const int kc = (int)((k + TILE_K - 1) / TILE_K);
    QMM_CUDA(launch_pack_x(x_dev, m, k, kc, static_cast<uint8_t*>(packed_dev), static_cast<cudaStream_t>(stream_v)));
    return QMM_OK;
}

}  // extern "C"

namespace {

XPackView xpack_view(const void* packed_dev, int kc, int m)
{
    XPackView xp;
    xp.base = static_cast<const uint8_t*>(packed_dev);
    xp.kc = kc;
    xp.ncp = xpack_ncp(m);
    return xp;
}

int gemv_packed_impl(const char* who, const qmm_weight* w, const void* packed_dev, float* y_dev, int m,
                     const PeerScatter* scatter, const GemvFuse* fuse, void* stream_v)
{
    if (int rc = check_weight(w, who)) {
        return rc;
    }
    const bool y_optional = fuse && (fuse->mode == EPI_RESID_PACK || fuse->mode == EPI_SWIGLU_PACK);
    const bool x_is_f32 = fuse && fuse->x_f32 != nullptr;
    if ((!packed_dev && !x_is_f32) || (!y_dev && !y_optional)) {
        return fail(QMM_E_INVALID, "%s: null activation or output pointer", who);
    }
    if (m < 1 || m > QMM_GEMV_MAX_BATCH) {
        return fail(QMM_E_INVALID, "%s: batch %d outside 1..%d", who, m, QMM_GEMV_MAX_BATCH);
    }
    if ((reinterpret_cast<uintptr_t>(packed_dev) & 15u) != 0) {
        return fail(QMM_E_INVALID, "%s: packed buffer must be 16-byte aligned", who);
    }
    DeviceGuard guard(w->device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    int* status = nullptr;
    if (int rc = get_status_word(w->device, &status)) {
        return rc;
    }
    const PeerScatter none = {};
    const GemvFuse plain = {};
    const cudaError_t e = launch_gemv_fused(view_of(w), xpack_view(packed_dev, w->kc, m), y_dev, m, status,
                                            scatter ? *scatter : none, fuse ? *fuse : plain,
                                            static_cast<cudaStream_t>(stream_v));
    if (e == cudaErrorInvalidValue) {
        return fail(QMM_E_INVALID, "%s: the weight's shape does not fit the requested fused form "
                    "(residual form: rows a multiple of 32; gate|up form: rows a multiple of 16, of 64 when packed; fp32 input: k a "
                    "multiple of 32; batch 1)", who);
    }
    if (e != cudaSuccess) {
        return fail_cuda(e, who);
    }
    return QMM_OK;
}

}  // namespace

int qmm_internal_status_word(int device, int** out)
{
    return get_status_word(device, out);
}

// For the decoder (llama_decoder.cu).
int qmm_internal_gemv_fused(const qmm_weight* w, const void* packed_dev, float* y_dev, const qmm::PeerScatter* scatter,
                            const qmm::GemvFuse* fuse, void* stream_v)
{
    return gemv_packed_impl("matvec", w, packed_dev, y_dev, 1, scatter, fuse, stream_v);
}

extern "C" {

int qmm_gemv_packed(const qmm_weight* w, const void* packed_dev, float* y_dev, int m, void* stream_v)
{
    return gemv_packed_impl("qmm_gemv_packed", w, packed_dev, y_dev, m, nullptr, nullptr, stream_v);
}

int qmm_gemv_packed_rms(const qmm_weight* w, const void* packed_dev, const double* ss_dev, int ss_count, int64_t d_in,
                        float eps, float* y_dev, void* stream_v)
{
    if (!ss_dev || ss_count < 1 || d_in < 1) {
        return fail(QMM_E_INVALID, "qmm_gemv_packed_rms: invalid sums of squares");
    }
    GemvFuse fu = {};
    fu.mode = EPI_STORE;
    fu.ss_in = ss_dev;
    fu.ss_count = ss_count;
    fu.d_in = (int)d_in;
    fu.eps = eps;
    return gemv_packed_impl("qmm_gemv_packed_rms", w, packed_dev, y_dev, 1, nullptr, &fu, stream_v);
}

int qmm_gemv_packed_residual(const qmm_weight* w, const void* packed_dev, float* h_dev, const float* norm_w_dev,
                             void* packed_out_dev, double* ss_out_dev, void* stream_v)
{
    if (!h_dev || !norm_w_dev || !packed_out_dev || !ss_out_dev) {
        return fail(QMM_E_INVALID, "qmm_gemv_packed_residual: null pointer");
    }
    GemvFuse fu = {};
    fu.mode = EPI_RESID_PACK;
    fu.h_in = h_dev;
    fu.h_out = h_dev;
    fu.norm_w = norm_w_dev;
    fu.ss_out = ss_out_dev;
    fu.packed_out = static_cast<uint8_t*>(packed_out_dev);
    return gemv_packed_impl("qmm_gemv_packed_residual", w, packed_dev, nullptr, 1, nullptr, &fu, stream_v);
}

int qmm_gemv_f32_residual(const qmm_weight* w, const float* x_dev, float* h_dev, const float* norm_w_dev,
                          void* packed_out_dev, double* ss_out_dev, void* stream_v)
{
    if (!x_dev || !h_dev || !norm_w_dev || !packed_out_dev || !ss_out_dev) {
        return fail(QMM_E_INVALID, "qmm_gemv_f32_residual: null pointer");
    }
    GemvFuse fu = {};
    fu.mode = EPI_RESID_PACK;
    fu.x_f32 = x_dev;
    fu.h_in = h_dev;
    fu.h_out = h_dev;
    fu.norm_w = norm_w_dev;
    fu.ss_out = ss_out_dev;
    fu.packed_out = static_cast<uint8_t*>(packed_out_dev);
    return gemv_packed_impl("qmm_gemv_f32_residual", w, nullptr, nullptr, 1, nullptr, &fu, stream_v);
}

int qmm_gemv_packed_swiglu(const qmm_weight* w_gate_up, const void* packed_dev, const double* ss_dev, int ss_count,
                           int64_t d_in, float eps, float* act_dev, void* stream_v)
{
    if (!act_dev || (ss_dev && (ss_count < 1 || d_in < 1))) {
        return fail(QMM_E_INVALID, "qmm_gemv_packed_swiglu: invalid argument");
    }
    GemvFuse fu = {};
    fu.mode = EPI_SWIGLU;
    fu.ss_in = ss_dev;
    fu.ss_count = ss_count;
    fu.d_in = (int)d_in;
    fu.eps = eps;
    return gemv_packed_impl("qmm_gemv_packed_swiglu", w_gate_up, packed_dev, act_dev, 1, nullptr, &fu, stream_v);
}

int qmm_gemv_packed_swiglu_pack(const qmm_weight* w_gate_up, const void* packed_dev, const double* ss_dev, int ss_count,
                                int64_t d_in, float eps, void* packed_out_dev, float* act_dev, void* stream_v)
{
    if (!packed_out_dev || (ss_dev && (ss_count < 1 || d_in < 1)) ||
        (reinterpret_cast<uintptr_t>(packed_out_dev) & 15u) != 0) {
        return fail(QMM_E_INVALID, "qmm_gemv_packed_swiglu_pack: invalid argument");
    }
    GemvFuse fu = {};
    fu.mode = EPI_SWIGLU_PACK;
    fu.ss_in = ss_dev;
    fu.ss_count = ss_count;
    fu.d_in = (int)d_in;
    fu.eps = eps;
    fu.packed_out = static_cast<uint8_t*>(packed_out_dev);
    return gemv_packed_impl("qmm_gemv_packed_swiglu_pack", w_gate_up, packed_dev, act_dev, 1, nullptr, &fu, stream_v);
}

int qmm_unpack_activations(int device, const void* packed_dev, int64_t k, float* x_dev, void* stream_v)
{
    if (!packed_dev || !x_dev || k < 1) {
        return fail(QMM_E_INVALID, "qmm_unpack_activations: invalid argument");
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    QMM_CUDA(launch_unpack_x(static_cast<const uint8_t*>(packed_dev), k, x_dev, static_cast<cudaStream_t>(stream_v)));
    return QMM_OK;
}

int qmm_gemv_f32(const qmm_weight* w, const float* x_dev, float* y_dev, int m, void* stream_v)
{
    if (int rc = check_weight(w, "qmm_gemv_f32")) {
        return rc;
    }
    if (!x_dev || !y_dev) {
        return fail(QMM_E_INVALID, "qmm_gemv_f32: null activation or output pointer");
    }
    if (m < 1 || m > QMM_GEMV_MAX_BATCH) {
        return fail(QMM_E_INVALID, "qmm_gemv_f32: batch %d outside 1..%d (use qmm_gemm_bf16 for prefill)", m,
                    QMM_GEMV_MAX_BATCH);
    }
    // Two activation buffers per (device, stream), used alternately.
    size_t one = 0;
    if (int rc = qmm_packed_activation_bytes(w->k, m, &one)) {
        return rc;
    }
    uint8_t* buf = nullptr;
    {
        DeviceGuard guard(w->device);
        if (!guard.ok) {
            return fail_cuda(guard.err, "cudaSetDevice");
        }
        if (int rc = get_workspace_half(w->device, stream_v, one, &buf)) {
            return rc;
        }
    }
    if (int rc = qmm_pack_activations(w->device, x_dev, m, w->k, buf, stream_v)) {
        return rc;
    }
    return qmm_gemv_packed(w, buf, y_dev, m, stream_v);
}

// ---- allocation-free variant ------------------------------------------------------------------
//
// The packed activations live in this file-scope device array (one instance per GPU
// that loads the library, held until exit).  In host code `g_static_scratch` is only a
// stand-in for the symbol, not a device address: the address each GPU gave the array
// is looked up once per device with cudaGetSymbolAddress and that pointer is what the
// kernels receive.  The last 256 bytes hold the status word of the bounded waits.
static __device__ __align__(256) unsigned char g_static_scratch[QMM_STATIC_SCRATCH_BYTES + 256];

namespace {
std::mutex g_static_mutex;
unsigned char* g_static_addr[64] = {};

// Device address of g_static_scratch on `device` (which must be current), and the status word the
// kernels of this path report to: the word the device already has (qmm_kernel_status reads exactly
// one word per device), else the array's tail, which then becomes the device's word.  No allocation.
int static_scratch_address(int device, unsigned char** out, int** status)
{
    if (device < 0 || device >= 64) {
        return fail(QMM_E_INVALID, "device index %d outside the 64 devices the static scratch table covers", device);
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) {
            return fail_cuda(e, "cudaGetSymbolAddress(static scratch)");
        }
        g_static_addr[device] = static_cast<unsigned char*>(p);
    }
    *out = g_static_addr[device];
    std::lock_guard<std::mutex> ws_lock(g_ws_mutex);
    auto it = g_status_words.find(device);
    if (it == g_status_words.end()) {
        // the array is zero-initialised when the module is loaded, so the word starts at 0
        it = g_status_words.emplace(device, reinterpret_cast<int*>(g_static_addr[device] + QMM_STATIC_SCRATCH_BYTES)).first;
    }
    *status = it->second;
    return QMM_OK;
}
}  // namespace

extern "C" int qmm_gemv_f32_static(const qmm_weight* w, const float* x_dev, float* y_dev, int m, void* stream_v)
{
    if (int rc = check_weight(w, "qmm_gemv_f32_static")) {
        return rc;
    }
    if (!x_dev || !y_dev) {
        return fail(QMM_E_INVALID, "qmm_gemv_f32_static: null activation or output pointer");
    }
    if (m < 1 || m > QMM_GEMV_MAX_BATCH) {
        return fail(QMM_E_INVALID, "qmm_gemv_f32_static: batch %d outside 1..%d", m, QMM_GEMV_MAX_BATCH);
    }
    const int ncp = xpack_ncp(m);
    const size_t need = m == 1 ? xpack1_bytes(w->kc) : xpack_bytes(w->kc, ncp);
    if (need > (size_t)QMM_STATIC_SCRATCH_BYTES) {
        return fail(QMM_E_INVALID,
                    "qmm_gemv_f32_static: packed activations for k=%lld, m=%d need %zu bytes, the fixed scratch holds %d; "
                    "use qmm_gemv_f32",
                    (long long)w->k, m, need, QMM_STATIC_SCRATCH_BYTES);
    }
    DeviceGuard guard(w->device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    unsigned char* buf = nullptr;
    int* status = nullptr;
    if (int rc = static_scratch_address(w->device, &buf, &status)) {
        return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    // pack_x_kernel rewrites every byte the matvec reads, so nothing of the previous call survives
    QMM_CUDA(launch_pack_x(x_dev, m, w->k, w->kc, buf, stream));
    QMM_CUDA(launch_gemv(view_of(w), xpack_view(buf, w->kc, m), y_dev, m, status, stream));
    return QMM_OK;
}

int qmm_gemv_f32_host(const qmm_weight* w, const float* x_host, float* y_host, int m, void* stream_v)
{
    if (int rc = check_weight(w, "qmm_gemv_f32_host")) {
        return rc;
    }
    if (!x_host || !y_host) {
        return fail(QMM_E_INVALID, "qmm_gemv_f32_host: null activation or output pointer");
    }
    if (m < 1 || m > QMM_GEMV_MAX_BATCH) {
        return fail(QMM_E_INVALID, "qmm_gemv_f32_host: batch %d outside 1..%d", m, QMM_GEMV_MAX_BATCH);
    }
    DeviceGuard guard(w->device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const size_t xb = (size_t)m * w->k * sizeof(float);
    const size_t yb = (size_t)m * w->n * sizeof(float);
    float* dx = nullptr;
    float* dy = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        Workspace& ws = g_workspaces[std::make_pair(w->device, stream_v)];
        if (ws.stage_x_bytes < xb) {
            if (ws.stage_x) {
                QMM_CUDA(cudaStreamSynchronize(stream));
                QMM_CUDA(cudaFree(ws.stage_x));
                ws.stage_x = nullptr;
                ws.stage_x_bytes = 0;
            }
            QMM_CUDA(cudaMalloc(&ws.stage_x, xb));
            ws.stage_x_bytes = xb;
        }
        if (ws.stage_y_bytes < yb) {
            if (ws.stage_y) {
                QMM_CUDA(cudaStreamSynchronize(stream));
                QMM_CUDA(cudaFree(ws.stage_y));
                ws.stage_y = nullptr;
                ws.stage_y_bytes = 0;
            }
            QMM_CUDA(cudaMalloc(&ws.stage_y, yb));
            ws.stage_y_bytes = yb;
        }
        dx = ws.stage_x;
        dy = ws.stage_y;
    }
    QMM_CUDA(cudaMemcpyAsync(dx, x_host, xb, cudaMemcpyHostToDevice, stream));
    if (int rc = qmm_gemv_f32(w, dx, dy, m, stream_v)) {
        return rc;
    }
    QMM_CUDA(cudaMemcpyAsync(y_host, dy, yb, cudaMemcpyDeviceToHost, stream));
    QMM_CUDA(cudaStreamSynchronize(stream));
    return QMM_OK;
}

int qmm_gemm_bf16(const qmm_weight* w, const void* x_bf16_dev, void* y_dev, int64_t m, int out_dtype, void* stream)
{
    if (int rc = check_weight(w, "qmm_gemm_bf16")) {
        return rc;
    }
    if (!x_bf16_dev || !y_dev) {
        return fail(QMM_E_INVALID, "qmm_gemm_bf16: null activation or output pointer");
    }
    if (m < 1) {
        return fail(QMM_E_INVALID, "qmm_gemm_bf16: invalid row count %lld", (long long)m);
    }
    if (out_dtype != QMM_OUT_F32 && out_dtype != QMM_OUT_BF16) {
        return fail(QMM_E_INVALID, "qmm_gemm_bf16: unknown output type %d", out_dtype);
    }
    DeviceGuard guard(w->device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    int* status = nullptr;
    if (int rc = get_status_word(w->device, &status)) {
        return rc;
    }
    const char* why = nullptr;
    cudaError_t e = launch_gemm_bf16(view_of(w), x_bf16_dev, y_dev, m, out_dtype == QMM_OUT_BF16 ? 1 : 0, w->sm_count,
                                     status, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess) {
        if (why) {
            return fail(e == cudaErrorNotSupported ? QMM_E_UNSUPPORTED : QMM_E_INVALID, "qmm_gemm_bf16: %s", why);
        }
        return fail_cuda(e, "qmm_gemm_bf16 launch");
    }
    return QMM_OK;
}

int qmm_gemm_f32(const qmm_weight* w, const float* x_dev, float* y_dev, int64_t m, void* stream_v)
{
    if (int rc = check_weight(w, "qmm_gemm_f32")) {
        return rc;
    }
    if (!x_dev || !y_dev || m < 1) {
        return fail(QMM_E_INVALID, "qmm_gemm_f32: null pointer or invalid row count");
    }
    DeviceGuard guard(w->device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const size_t need = (size_t)m * (size_t)w->k * 2;
    void* conv = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        Workspace& ws = g_workspaces[std::make_pair(w->device, stream_v)];
        if (ws.conv_bytes < need) {
            if (ws.conv) {
                QMM_CUDA(cudaStreamSynchronize(stream));
                QMM_CUDA(cudaFree(ws.conv));
                ws.conv = nullptr;
                ws.conv_bytes = 0;
            }
            QMM_CUDA(cudaMalloc(&ws.conv, align_up(need, 1 << 20)));
            ws.conv_bytes = align_up(need, 1 << 20);
        }
        conv = ws.conv;
    }
    QMM_CUDA(launch_f32_to_bf16(x_dev, m * w->k, conv, stream));
    return qmm_gemm_bf16(w, conv, y_dev, m, QMM_OUT_F32, stream_v);
}

int qmm_kernel_status(int device, int* status_out)
{
    if (!status_out) {
        return fail(QMM_E_INVALID, "status_out is null");
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    int* word = nullptr;
    if (int rc = get_status_word(device, &word)) {
        return rc;
    }
    QMM_CUDA(cudaMemcpy(status_out, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status_out != 0) {
        QMM_CUDA(cudaMemset(word, 0, sizeof(int)));
        return fail(QMM_E_KERNEL, "a kernel gave up on a bounded wait (status %d); its output is invalid",
                    *status_out);
    }
    return QMM_OK;
}

int qmm_stream_synchronize(int device, void* stream)
{
    DeviceGuard guard(device);
    if (!guard.ok) {
        return fail_cuda(guard.err, "cudaSetDevice");
    }
    QMM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return QMM_OK;
}

int qmm_release_workspaces(void)
{
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    int rc = QMM_OK;
    for (auto& kv : g_workspaces) {
        DeviceGuard guard(kv.first.first);
        Workspace& ws = kv.second;
        for (void* p : {static_cast<void*>(ws.base), static_cast<void*>(ws.stage_x), static_cast<void*>(ws.stage_y), ws.conv}) {
            if (p && cudaFree(p) != cudaSuccess) {
                rc = fail(QMM_E_CUDA, "cudaFree(workspace) failed");
            }
        }
    }
    g_workspaces.clear();
    return rc;
}

}  // extern "C"

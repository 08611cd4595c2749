// Glue kernels of the LLaMA decoder around the quantized linears: embedding row
// dequantization, RMSNorm, interleaved RoPE, fp16 KV cache, attention, SwiGLU, residual
// adds and greedy argmax.  Semantics follow the reference graph builders:
//   RMSNorm   x / sqrt(mean(x^2) + eps) * w, statistics in double
//             (src/LiteNN/ComputePrimitives.h:795-821)
//   RoPE      interleaved pairs (x[2i], x[2i+1]), angle = pos * theta^(-2i/d), tables made in
//             double and cast to fp32, rotation in fp32 (src/LiteNN/Layer/RoPE.h:22-114)
//   attention scores = q.k * 1/sqrt(head_dim), causal, max-shifted softmax, probs.V
//             (src/LiteNN/Layer/FlashAttnExt.h:100-229; tools/gguf/LLaMABuilder.cpp:350-404);
//             GQA maps head h to kv head h / (heads / kv_heads) (LLaMABuilder.cpp:524)
//   SwiGLU    down(silu(gate(x)) * up(x)), silu(x) = x / (1 + exp(-x))
//             (src/LiteNN/Layer/SwiGLU.h:54-64; Layer/Activation.h:20-33,52-59)
// The KV cache holds rotated keys and values as fp16 (the benchmark configuration's choice;
// the reference keeps them in the model dtype, LLaMABuilder.cpp:847-849).
// These kernels are latency-sized (one token of a 4096-wide model); the weight streaming
// lives in qmm_gemv.cu / qmm_gemm.cu.
#include <cuda_bf16.h>
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "llama_device.cuh"
#include "llama_kernels.h"
#include "qmm_layout.cuh"

namespace qmm {

namespace {

__device__ __forceinline__ void pdl_trigger()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_sync()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ double block_sum_double(double v, double* red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    }
    __syncthreads();
    if (lane == 0) {
        red[warp] = v;
    }
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nw; ++i) {
        t += red[i];
    }
    return t;
}

// ---- decode (one token) -------------------------------------------------------------------------

// h[d] = dequantized row `token` of the raw (not repacked) embedding payload.
__global__ void embed_row_kernel(int fmt, const uint8_t* __restrict__ raw, const int* __restrict__ tokens, int n_rows,
                                 int d, float* __restrict__ h)
{
    pdl_trigger();
    pdl_sync();
    const int elems = block_elems(fmt), bytes = block_bytes(fmt);
    const int64_t row_bytes = (int64_t)(d / elems) * bytes;
    for (int r = blockIdx.y; r < n_rows; r += gridDim.y) {
        const uint8_t* row = raw + (int64_t)tokens[r] * row_bytes;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < d; i += gridDim.x * blockDim.x) {
            h[(int64_t)r * d + i] = dequant_raw_element(fmt, row + (i / elems) * bytes, i % elems);
        }
    }
}

// h_out = h_in + add (add optional); xn = rmsnorm(h_out) * w; packed = pack(xn).
// One CTA per 256-wide chunk: every CTA sums the squares of the whole row itself (the row is a
// few KB in L2), then normalizes, packs and stores only its own chunk, so nothing crosses CTAs.
// h_out must not alias h_in (other CTAs still read h_in); it may be null.
//
// Tensor-parallel form (pg.tp_size > 1): `add` is only this rank's addend.  The other ranks'
// addends arrive in pg.recv as {value, exchange number} packets stored by their matvec kernels
// (PeerScatter, qmm_common.cuh).  A reader polls a packet until it carries this exchange's
// number (bounded), and adds the addends in rank order, so every rank computes bit-identical
// sums without a separate all-reduce launch.

__device__ __forceinline__ uint4 ld_sys_v4(const uint2* p)
{
    uint4 q;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                 : "l"(p)
                 : "memory");
    return q;
}

// Sum over the ranks of elements 4*i4 .. 4*i4+3, own addend at its place in the rank order.
// The packets of all peers are requested at once (two 16-byte loads per peer), then checked;
// only a packet that has not arrived yet is polled again (bounded).
__device__ __forceinline__ float4 peer_sum4(const PeerGather& pg, const float* add, int d, int i4, unsigned int epoch,
                                            bool& ok)
{
    constexpr int MAXP = 7;
    const int np = pg.tp_size - 1;
    uint4 lo[MAXP], hi[MAXP];
#pragma unroll
    for (int p = 0; p < MAXP; ++p) {
        if (p < np) {
            const uint2* src = pg.recv + (size_t)(p + (p >= pg.tp_rank ? 1 : 0)) * d + 4 * i4;
            lo[p] = ld_sys_v4(src);
            hi[p] = ld_sys_v4(src + 2);
        }
    }
#pragma unroll
    for (int p = 0; p < MAXP; ++p) {
        if (p < np) {
            const uint2* src = pg.recv + (size_t)(p + (p >= pg.tp_rank ? 1 : 0)) * d + 4 * i4;
            unsigned int spin = 0;
            while (ok && !(lo[p].y == epoch && lo[p].w == epoch && hi[p].y == epoch && hi[p].w == epoch)) {
                if (++spin > (1u << 21)) {
                    ok = false;
                    atomicExch(pg.status, 5);  // a peer's addend never came; the sum is incomplete
                    break;
                }
                lo[p] = ld_sys_v4(src);
                hi[p] = ld_sys_v4(src + 2);
            }
        }
    }
    const float4 own = reinterpret_cast<const float4*>(add)[i4];
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < MAXP; ++p) {  // peers in rank order; the own addend goes in before peer index tp_rank
        if (p == pg.tp_rank) {
            a.x += own.x;
            a.y += own.y;
            a.z += own.z;
            a.w += own.w;
        }
        if (p < np) {
            a.x += __uint_as_float(lo[p].x);
            a.y += __uint_as_float(lo[p].z);
            a.z += __uint_as_float(hi[p].x);
            a.w += __uint_as_float(hi[p].z);
        }
    }
    if (pg.tp_rank == MAXP) {  // rank 7 of 8: after every peer
        a.x += own.x;
        a.y += own.y;
        a.z += own.z;
        a.w += own.w;
    }
    return a;
}

template <bool TP>
__global__ void __launch_bounds__(256) resid_rmsnorm_pack_kernel(const float* __restrict__ h_in,
                                                                 const float* __restrict__ add,
                                                                 const float* __restrict__ w, float eps, int d,
                                                                 uint8_t* __restrict__ packed,
                                                                 float* __restrict__ h_out, PeerGather pg)
{
    __shared__ double red[8];
    __shared__ float vals[256];
    __shared__ float4 sums[TP ? 64 : 1];  // this CTA's chunk of the summed addend (tensor-parallel form)
    pdl_trigger();
    const bool tp = TP && add != nullptr;
    unsigned int epoch = 0;
    bool ok = true;
    if (tp) {  // the position was set by an earlier token
        epoch = (unsigned int)(*pg.pos * pg.sites + pg.site + 1);
    }
    pdl_sync();
    if (tp) {
        ok = *reinterpret_cast<volatile int*>(pg.status) == 0;  // after one timeout nothing waits again
    }
    const int c = blockIdx.x, kc = (d + 255) / 256;
    double ss = 0.0;
    const int n4 = d >> 2;  // d is a multiple of 32 (block formats)
    for (int i = threadIdx.x; i < n4; i += 256) {
        float4 v = reinterpret_cast<const float4*>(h_in)[i];
        if (add) {
            const float4 a = tp ? peer_sum4(pg, add, d, i, epoch, ok) : reinterpret_cast<const float4*>(add)[i];
            if (tp && (i >> 6) == c) {
                sums[i & 63] = a;
            }
            v.x += a.x;
            v.y += a.y;
            v.z += a.z;
            v.w += a.w;
        }
        ss += (double)v.x * (double)v.x + (double)v.y * (double)v.y;
        ss += (double)v.z * (double)v.z + (double)v.w * (double)v.w;
    }
    ss = block_sum_double(ss, red);  // (also orders the writes of `sums` before the reads below)
    const int idx = c * 256 + threadIdx.x;
    float mine = 0.0f;
    if (idx < d) {
        mine = h_in[idx];
        if (add) {
            mine += tp ? reinterpret_cast<const float*>(sums)[threadIdx.x] : add[idx];
        }
        if (h_out) {
            h_out[idx] = mine;
        }
    }
    const double inv = 1.0 / sqrt(ss / (double)d + (double)eps);
    vals[threadIdx.x] = idx < d ? (float)((double)mine * inv) * w[idx] : 0.0f;
    __syncthreads();
    if (threadIdx.x < 32) {
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r[i] = vals[8 * threadIdx.x + i];
        }
        warp_pack_chunk(r, c, kc, packed);
    }
}

constexpr int NORM_CLUSTER = 8;   // CTAs of the tensor-parallel norm kernel (one cluster)
constexpr int NORM_MAXJ = 4;      // chunks per CTA it can hold: d_model <= 8 * 4 * 256

// Tensor-parallel form of resid_rmsnorm_pack_kernel for d <= 8192, as ONE cluster of 8 CTAs.
// CTA `rank` owns chunks rank, rank + 8, ...; it gathers only those chunks' packets from the
// peers (every (position, rank group) pair has its own thread, so all packet loads of the CTA
// are in flight together), the CTAs exchange their partial sums of squares through distributed
// shared memory, and each CTA normalizes and packs its chunks.  Against the one-CTA-per-chunk
// form, which makes every CTA read every peer's whole addend, this removes 15/16 of the polling.
// The addends are added in a fixed association — ranks r = g, g + 4 ascending inside group
// g = r mod 4, then ((S0 + S1) + S2) + S3 — with the own addend in its rank's place, so all
// ranks compute bit-identical sums.
__global__ void __launch_bounds__(256) resid_rmsnorm_pack_tp_kernel(const float* __restrict__ h_in,
                                                                    const float* __restrict__ add,
                                                                    const float* __restrict__ w, float eps, int d,
                                                                    uint8_t* __restrict__ packed,
                                                                    float* __restrict__ h_out, PeerGather pg)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float4 part[NORM_MAXJ][4][64];  // [chunk slot][rank group][position]
    __shared__ float vals[NORM_MAXJ][256];
    __shared__ double red[8];
    __shared__ double cl_ss[NORM_CLUSTER];     // every CTA's sum of squares, written by its owner
    pdl_trigger();
    const int rank = (int)cluster.block_rank();
    const int kc = (d + 255) / 256;
    const int t = threadIdx.x, pos = t & 63, grp = t >> 6;
    const unsigned int epoch = (unsigned int)(*pg.pos * pg.sites + pg.site + 1);  // set by an earlier token
    pdl_sync();
    bool ok = *reinterpret_cast<volatile int*>(pg.status) == 0;  // after one timeout nothing waits again

    // 1. request every packet this thread is responsible for, then settle them
    uint4 lo[NORM_MAXJ][2], hi[NORM_MAXJ][2];
#pragma unroll
    for (int j = 0; j < NORM_MAXJ; ++j) {
        const int c = rank + NORM_CLUSTER * j;
        const int e0 = c * 256 + 4 * pos;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int r = grp + 4 * q;
            if (c < kc && e0 < d && r < pg.tp_size && r != pg.tp_rank) {
                const uint2* src = pg.recv + (size_t)r * d + e0;
                lo[j][q] = ld_sys_v4(src);
                hi[j][q] = ld_sys_v4(src + 2);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NORM_MAXJ; ++j) {
        const int c = rank + NORM_CLUSTER * j;
        const int e0 = c * 256 + 4 * pos;
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int r = grp + 4 * q;
            if (c < kc && e0 < d && r < pg.tp_size) {
                float4 a;
                if (r == pg.tp_rank) {
                    a = *reinterpret_cast<const float4*>(add + e0);
                } else {
                    const uint2* src = pg.recv + (size_t)r * d + e0;
                    unsigned int spin = 0;
                    while (ok && !(lo[j][q].y == epoch && lo[j][q].w == epoch && hi[j][q].y == epoch &&
                                   hi[j][q].w == epoch)) {
                        if (++spin > (1u << 21)) {
                            ok = false;
                            atomicExch(pg.status, 5);  // a peer's addend never came; the sum is incomplete
                            break;
                        }
                        lo[j][q] = ld_sys_v4(src);
                        hi[j][q] = ld_sys_v4(src + 2);
                    }
                    a = make_float4(__uint_as_float(lo[j][q].x), __uint_as_float(lo[j][q].z), __uint_as_float(hi[j][q].x),
                                    __uint_as_float(hi[j][q].z));
                }
                s4.x += a.x;
                s4.y += a.y;
                s4.z += a.z;
                s4.w += a.w;
            }
        }
        part[j][grp][pos] = s4;
    }
    __syncthreads();

    // 2. residual add, sum of squares over the cluster
    float mine[NORM_MAXJ];
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < NORM_MAXJ; ++j) {
        const int c = rank + NORM_CLUSTER * j;
        const int idx = c * 256 + t;
        mine[j] = 0.0f;
        if (c < kc && idx < d) {
            const float* p0 = reinterpret_cast<const float*>(&part[j][0][0]);
            const float a = ((p0[t] + p0[256 + t]) + p0[512 + t]) + p0[768 + t];
            mine[j] = h_in[idx] + a;
            if (h_out) {
                h_out[idx] = mine[j];
            }
            ss += (double)mine[j] * (double)mine[j];
        }
    }
    ss = block_sum_double(ss, red);
    if (t < NORM_CLUSTER) {
        *cluster.map_shared_rank(&cl_ss[rank], t) = ss;  // my sum into CTA t's table
    }
    cluster.sync();
    double total = 0.0;
#pragma unroll
    for (int r = 0; r < NORM_CLUSTER; ++r) {
        total += cl_ss[r];
    }
    const double inv = 1.0 / sqrt(total / (double)d + (double)eps);

    // 3. normalize and pack this CTA's chunks: warp j packs chunk slot j
#pragma unroll
    for (int j = 0; j < NORM_MAXJ; ++j) {
        const int idx = (rank + NORM_CLUSTER * j) * 256 + t;
        vals[j][t] = idx < d ? (float)((double)mine[j] * inv) * w[idx] : 0.0f;
    }
    __syncthreads();
    const int wj = t >> 5, lane = t & 31;
    if (wj < NORM_MAXJ && rank + NORM_CLUSTER * wj < kc) {
        float r8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r8[i] = vals[wj][8 * lane + i];
        }
        warp_pack_chunk(r8, rank + NORM_CLUSTER * wj, kc, packed);
    }
}

// cos/sin tables [max_seq][rope_dim/2], computed in double and cast (Layer/RoPE.h:22-39).
__global__ void rope_table_kernel(int max_seq, int rope_dim, double theta, float* __restrict__ rope_cos,
                                  float* __restrict__ rope_sin)
{
    const int half = rope_dim / 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (int64_t)max_seq * half;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int pos = (int)(i / half), dim = (int)(i % half);
        const double inv_freq = pow(theta, -2.0 * (double)dim / (double)rope_dim);
        const double ang = (double)pos * inv_freq;
        rope_cos[i] = (float)cos(ang);
        rope_sin[i] = (float)sin(ang);
    }
}

// RoPE on q and k of one token at position *pos, K/V appended to the fp16 cache.
//   qkv: [n_heads*hd | n_kv*hd | n_kv*hd] fp32 (q rotated in place)
//   cache_k / cache_v: [n_kv][max_seq][hd] fp16
__global__ void rope_kv_kernel(float* __restrict__ qkv, const int* __restrict__ pos_ptr, int pos_add, int n_heads,
                               int n_kv, int hd, int rope_dim, const float* __restrict__ rope_cos,
                               const float* __restrict__ rope_sin, int max_seq, __half* __restrict__ cache_k,
                               __half* __restrict__ cache_v, int row_stride)
{
    pdl_trigger();
    pdl_sync();
    const int row = blockIdx.y;  // token within the batch (prefill) or 0
    const int pos = *pos_ptr + pos_add + row;
    float* base = qkv + (int64_t)row * row_stride;
    const int pairs_q = n_heads * hd / 2, pairs_k = n_kv * hd / 2;
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < pairs_q + pairs_k + n_kv * hd; p += gridDim.x * blockDim.x) {
        if (p < pairs_q + pairs_k) {
            const bool is_k = p >= pairs_q;
            const int pp = is_k ? p - pairs_q : p;
            const int head = pp / (hd / 2), i = pp % (hd / 2);
            float* x = base + (is_k ? n_heads * hd : 0) + head * hd + 2 * i;
            float a = x[0], b = x[1];
            if (2 * i < rope_dim) {
                const float c = rope_cos[(int64_t)pos * (rope_dim / 2) + i];
                const float s = rope_sin[(int64_t)pos * (rope_dim / 2) + i];
                const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
                const float rb = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
                a = ra;
                b = rb;
            }
            if (is_k) {
                __half* dst = cache_k + ((int64_t)head * max_seq + pos) * hd + 2 * i;
                dst[0] = __float2half_rn(a);
                dst[1] = __float2half_rn(b);
            } else {
                x[0] = a;
                x[1] = b;
            }
        } else {
            const int e = p - pairs_q - pairs_k;
            const int head = e / hd, i = e % hd;
            cache_v[((int64_t)head * max_seq + pos) * hd + i] = __float2half_rn(base[(n_heads + n_kv) * hd + e]);
        }
    }
}

constexpr int ATTN_CLUSTER = 8;  // CTAs per 256-wide context chunk (portable cluster size)

// Decode attention of one token in one launch: RoPE of q and of the new key, K/V append to
// the fp16 cache, attention over the cache, merge and activation packing.
// A cluster of CTAs owns one 256-wide chunk of the context vector (256/hd heads).  Inside a
// CTA warp w serves head (w % HH) of the chunk and key split (rank * NSUB + w / HH); every warp
// rotates its own copy of q, takes batches of 8 cached keys (all loads of a batch are issued
// before any use) and keeps an online softmax.  The last split also takes the new position,
// whose key and value come straight from the qkv vector (rounded to fp16 as the cache holds
// them) and are stored to the cache by the first head of each kv group.  Partials are merged
// per CTA in shared memory and stored into rank 0's shared memory (distributed shared memory);
// rank 0 merges the CTAs' partials and writes the packed chunk.
template <int DPL>  // head dims per lane = hd / 32 (2 or 4)
__global__ void __launch_bounds__(256) attn_fused_kernel(const float* __restrict__ qkv, const int* __restrict__ pos_ptr,
                                                         int n_heads, int n_kv, int rope_dim,
                                                         const float* __restrict__ rope_cos,
                                                         const float* __restrict__ rope_sin, int max_seq,
                                                         __half* __restrict__ cache_k, __half* __restrict__ cache_v,
                                                         uint8_t* __restrict__ packed)
{
    constexpr int hd = 32 * DPL;
    constexpr int HH = 256 / hd;  // heads per chunk
    constexpr int NSUB = 8 / HH;  // key splits per CTA
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    // Shared memory is kept small (13 KB) on purpose: this kernel is launched while the qkv matvec
    // still fills the SMs, and it can only start its preloads early if a CTA fits beside them.
    __shared__ float sm[8][hd + 2];                      // per-warp partials of this CTA
    __shared__ float parts[ATTN_CLUSTER][HH][hd + 2];    // rank 0's copy collects every CTA's merged partials
    __shared__ float vals[256];
    pdl_trigger();
    // Everything up to pdl_sync() reads only what earlier tokens left behind (the position, the
    // rotation tables, the cached keys and values), so it runs while the qkv GEMV is finishing.
    const int rank = (int)cluster.block_rank();
    const int chunk = blockIdx.x / ATTN_CLUSTER;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hl = warp % HH, sub = warp / HH;
    const int head = chunk * HH + hl;
    const int nsplit = ATTN_CLUSTER * NSUB, split = rank * NSUB + sub;
    const int pos = *pos_ptr;
    const int per = (pos + nsplit - 1) / nsplit;
    const int k0 = split * per, k1 = min(pos, k0 + per);
    const int group = n_heads / n_kv, kvh = head < n_heads ? head / group : 0;
    const __half* kb = cache_k + (int64_t)kvh * max_seq * hd + lane * DPL;
    const __half* vb = cache_v + (int64_t)kvh * max_seq * hd + lane * DPL;
    float cs_[DPL / 2], sn_[DPL / 2];
#pragma unroll
    for (int j = 0; j < DPL / 2; ++j) {
        const int i = lane * (DPL / 2) + j;
        const bool rot = 2 * i < rope_dim;
        cs_[j] = rot ? rope_cos[(int64_t)pos * (rope_dim / 2) + i] : 1.0f;
        sn_[j] = rot ? rope_sin[(int64_t)pos * (rope_dim / 2) + i] : 0.0f;
    }
    // The first 16 keys of this warp's split go to registers now; longer splits are prefetched
    // to L2 and loaded in the loop below.
    KvBatch<DPL> pre0, pre1;
    if (head < n_heads) {
        kv_batch_load<DPL>(pre0, kb, vb, k0, k1);
        kv_batch_load<DPL>(pre1, kb, vb, k0 + 8, k1);
        // one 128-byte line per lane and step: this warp's rows of K and of V are contiguous
        const char* kl = reinterpret_cast<const char*>(cache_k + ((int64_t)kvh * max_seq + k0 + 16) * hd);
        const char* vl = reinterpret_cast<const char*>(cache_v + ((int64_t)kvh * max_seq + k0 + 16) * hd);
        const int bytes = (k1 - k0 - 16) * hd * (int)sizeof(__half);
        for (int o = lane * 128; o < bytes; o += 32 * 128) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(kl + o));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(vl + o));
        }
    }
    pdl_sync();
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    if (head < n_heads) {
        const float scale = rsqrtf((float)hd);
        const bool takes_new = split == nsplit - 1;
        float2 qx[DPL / 2], kx[DPL / 2], vx[DPL / 2];
#pragma unroll
        for (int j = 0; j < DPL / 2; ++j) {
            qx[j] = *reinterpret_cast<const float2*>(qkv + head * hd + lane * DPL + 2 * j);
            if (takes_new) {
                kx[j] = *reinterpret_cast<const float2*>(qkv + (n_heads + kvh) * hd + lane * DPL + 2 * j);
                vx[j] = *reinterpret_cast<const float2*>(qkv + (n_heads + n_kv + kvh) * hd + lane * DPL + 2 * j);
            }
        }
        float qv[DPL];
#pragma unroll
        for (int j = 0; j < DPL / 2; ++j) {
            const float2 x = qx[j];
            const bool rot = 2 * (lane * (DPL / 2) + j) < rope_dim;
            const float ra = rot ? __fsub_rn(__fmul_rn(x.x, cs_[j]), __fmul_rn(x.y, sn_[j])) : x.x;
            const float rb = rot ? __fadd_rn(__fmul_rn(x.x, sn_[j]), __fmul_rn(x.y, cs_[j])) : x.y;
            qv[2 * j] = ra * scale;
            qv[2 * j + 1] = rb * scale;
        }
        kv_batch_apply<DPL>(pre0, qv, k0, k1, m, l, acc);
        kv_batch_apply<DPL>(pre1, qv, k0 + 8, k1, m, l, acc);
        for (int kbase = k0 + 16; kbase < k1; kbase += 8) {
            KvBatch<DPL> cur;
            kv_batch_load<DPL>(cur, kb, vb, kbase, k1);
            kv_batch_apply<DPL>(cur, qv, kbase, k1, m, l, acc);
        }
        if (takes_new) {  // the new position
            __half kn[DPL], vn[DPL];
#pragma unroll
            for (int j = 0; j < DPL / 2; ++j) {
                const float2 x = kx[j];
                const float2 v = vx[j];
                const bool rot = 2 * (lane * (DPL / 2) + j) < rope_dim;
                const float ra = rot ? __fsub_rn(__fmul_rn(x.x, cs_[j]), __fmul_rn(x.y, sn_[j])) : x.x;
                const float rb = rot ? __fadd_rn(__fmul_rn(x.x, sn_[j]), __fmul_rn(x.y, cs_[j])) : x.y;
                kn[2 * j] = __float2half_rn(ra);
                kn[2 * j + 1] = __float2half_rn(rb);
                vn[2 * j] = __float2half_rn(v.x);
                vn[2 * j + 1] = __float2half_rn(v.y);
            }
            if (head % group == 0) {
                __half* kd = cache_k + ((int64_t)kvh * max_seq + pos) * hd + lane * DPL;
                __half* vd = cache_v + ((int64_t)kvh * max_seq + pos) * hd + lane * DPL;
#pragma unroll
                for (int i = 0; i < DPL; i += 2) {
                    *reinterpret_cast<__half2*>(kd + i) = *reinterpret_cast<const __half2*>(&kn[i]);
                    *reinterpret_cast<__half2*>(vd + i) = *reinterpret_cast<const __half2*>(&vn[i]);
                }
            }
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                dot += qv[i] * __half2float(kn[i]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
            }
            const float mb = fmaxf(m, dot);
            const float corr = __expf(m - mb), p = __expf(dot - mb);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                acc[i] = acc[i] * corr + p * __half2float(vn[i]);
            }
            m = mb;
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        sm[warp][lane * DPL + i] = acc[i];
    }
    if (lane == 0) {
        sm[warp][hd] = m;
        sm[warp][hd + 1] = l;
    }
    __syncthreads();
    {   // merge this CTA's key splits per head and hand the result to rank 0 of the cluster
        const int h2 = threadIdx.x / hd, e = threadIdx.x % hd;
        float M = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < NSUB; ++s2) {
            M = fmaxf(M, sm[h2 + HH * s2][hd]);
        }
        float a = 0.0f, L = 0.0f;
#pragma unroll
        for (int s2 = 0; s2 < NSUB; ++s2) {
            const float mw = sm[h2 + HH * s2][hd];
            const float f = mw == -INFINITY ? 0.0f : __expf(mw - M);
            a += sm[h2 + HH * s2][e] * f;
            L += sm[h2 + HH * s2][hd + 1] * f;
        }
        float* dst = cluster.map_shared_rank(&parts[0][0][0], 0) + (rank * HH + h2) * (hd + 2);
        dst[e] = a;
        if (e == 0) {
            dst[hd] = M;
            dst[hd + 1] = L;
        }
    }
    cluster.sync();  // remote stores above are visible to rank 0 after this
    if (rank != 0) {
        return;
    }
    {
        const int h2 = threadIdx.x / hd, e = threadIdx.x % hd;
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < ATTN_CLUSTER; ++r) {
            M = fmaxf(M, parts[r][h2][hd]);
        }
        float a = 0.0f, L = 0.0f;
#pragma unroll
        for (int r = 0; r < ATTN_CLUSTER; ++r) {
            const float mp = parts[r][h2][hd];
            const float f = mp == -INFINITY ? 0.0f : __expf(mp - M);
            a += parts[r][h2][e] * f;
            L += parts[r][h2][hd + 1] * f;
        }
        vals[threadIdx.x] = L > 0.0f ? a / L : 0.0f;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        float r8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r8[i] = vals[8 * threadIdx.x + i];
        }
        warp_pack_chunk(r8, chunk, (n_heads * hd + 255) / 256, packed);
    }
}

// act = silu(gate) * up, packed; grid = chunks of 256, one warp each.
__global__ void __launch_bounds__(32) silu_mul_pack_kernel(const float* __restrict__ gu, int ffn,
                                                           uint8_t* __restrict__ packed)
{
    pdl_trigger();
    pdl_sync();
    const int c = blockIdx.x, lane = threadIdx.x;
    const int kc = (ffn + 255) / 256;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = c * 256 + 8 * lane + i;
        if (idx < ffn) {
            const float g = gu[idx], u = gu[ffn + idx];
            v[i] = (g / (1.0f + expf(-g))) * u;
        } else {
            v[i] = 0.0f;
        }
    }
    warp_pack_chunk(v, c, kc, packed);
}

// Greedy argmax, first stage (lowest index wins ties): CTA b writes its (value bits, index)
// candidate to best_pair[2b..2b+1].
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int n, int index_offset,
                                                      int* __restrict__ best_pair)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_sync();
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = logits[i];
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) {
                bv = sv[w];
                bi = si[w];
            }
        }
        best_pair[2 * blockIdx.x] = __float_as_int(bv);
        best_pair[2 * blockIdx.x + 1] = bi == 0x7FFFFFFF ? bi : bi + index_offset;
    }
}

// Picks the winner among `ranks` (value, index) candidates, stores the token, advances pos.
__global__ void commit_token_kernel(const int* __restrict__ pairs, int ranks, int* __restrict__ token,
                                    int* __restrict__ pos, int* __restrict__ out_tokens, int* __restrict__ out_count)
{
    pdl_trigger();
    pdl_sync();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        float bv = __int_as_float(pairs[0]);
        int bi = pairs[1];
        for (int r = 1; r < ranks; ++r) {
            const float v = __int_as_float(pairs[2 * r]);
            const int i = pairs[2 * r + 1];
            if (v > bv || (v == bv && i < bi)) {
                bv = v;
                bi = i;
            }
        }
        *token = bi;
        out_tokens[*out_count] = bi;
        *out_count += 1;
        *pos += 1;
    }
}

// ---- prefill (many tokens) ------------------------------------------------------------------------

// Per row: h += add (optional); xn = bf16(rmsnorm(h) * w).
__global__ void __launch_bounds__(256) resid_rmsnorm_rows_kernel(float* __restrict__ h, const float* __restrict__ add,
                                                                 const float* __restrict__ w, float eps, int d,
                                                                 __nv_bfloat16* __restrict__ xn)
{
    __shared__ double red[32];
    const int64_t row = blockIdx.x;
    float* hr = h + row * d;
    double ss = 0.0;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = hr[i];
        if (add) {
            v += add[row * d + i];
            hr[i] = v;
        }
        ss += (double)v * (double)v;
    }
    ss = block_sum_double(ss, red);
    const double denom = sqrt(ss / (double)d + (double)eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        xn[row * d + i] = __float2bfloat16_rn((float)((double)hr[i] / denom) * w[i]);
    }
}

// Causal attention over the fp16 cache for rows 0..m-1 at positions pos0+row: one warp per
// (row, head), online softmax over keys 0..pos; output bf16 ctx[m][n_heads*hd].
__global__ void __launch_bounds__(128) attn_prefill_kernel(const float* __restrict__ qkv, int row_stride, int m,
                                                           int pos0, int n_heads, int n_kv, int hd, int max_seq,
                                                           const __half* __restrict__ cache_k,
                                                           const __half* __restrict__ cache_v,
                                                           __nv_bfloat16* __restrict__ ctx)
{
    const int lane = threadIdx.x & 31;
    const int64_t wid = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wid >= (int64_t)m * n_heads) {
        return;
    }
    const int row = (int)(wid / n_heads), head = (int)(wid % n_heads);
    const int kvh = head / (n_heads / n_kv);
    const int dpl = hd / 32;
    const float scale = rsqrtf((float)hd);
    float qv[8], acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        qv[i] = i < dpl ? qkv[(int64_t)row * row_stride + head * hd + lane * dpl + i] : 0.0f;
        acc[i] = 0.0f;
    }
    float mx = -INFINITY, l = 0.0f;
    const __half* kb = cache_k + (int64_t)kvh * max_seq * hd;
    const __half* vb = cache_v + (int64_t)kvh * max_seq * hd;
    const int n_keys = pos0 + row + 1;
    for (int k = 0; k < n_keys; ++k) {
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < dpl) {
                dot += qv[i] * __half2float(kb[(int64_t)k * hd + lane * dpl + i]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
        }
        const float s = dot * scale;
        const float mn = fmaxf(mx, s);
        const float corr = __expf(mx - mn), p = __expf(s - mn);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < dpl) {
                acc[i] = acc[i] * corr + p * __half2float(vb[(int64_t)k * hd + lane * dpl + i]);
            }
        }
        mx = mn;
    }
    for (int i = 0; i < dpl; ++i) {
        ctx[(int64_t)row * n_heads * hd + head * hd + lane * dpl + i] = __float2bfloat16_rn(acc[i] / l);
    }
}

// act[m][ffn] = bf16(silu(gate) * up) from gu[m][2*ffn].
__global__ void silu_mul_rows_kernel(const float* __restrict__ gu, int64_t m, int ffn, __nv_bfloat16* __restrict__ act)
{
    const int64_t total = m * ffn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / ffn;
        const int c = (int)(i % ffn);
        const float g = gu[r * 2 * ffn + c], u = gu[r * 2 * ffn + ffn + c];
        act[i] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * u);
    }
}

__global__ void add_rows_kernel(float* __restrict__ h, const float* __restrict__ add, int64_t total)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        h[i] += add[i];
    }
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, int cluster, cudaStream_t stream,
                               Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace

cudaError_t ll_rope_tables(int max_seq, int rope_dim, double theta, float* rope_cos, float* rope_sin, cudaStream_t st)
{
    rope_table_kernel<<<64, 256, 0, st>>>(max_seq, rope_dim, theta, rope_cos, rope_sin);
    return cudaGetLastError();
}

cudaError_t ll_embed_rows(int fmt, const uint8_t* raw, const int* tokens, int n_rows, int d, float* h, cudaStream_t st)
{
    return launch_pdl(embed_row_kernel, dim3((d + 255) / 256, n_rows < 1024 ? n_rows : 1024), dim3(256), 0, st, fmt,
                      raw, tokens, n_rows, d, h);
}

cudaError_t ll_resid_rmsnorm_pack(const float* h_in, const float* add, const float* w, float eps, int d,
                                  uint8_t* packed, float* h_out, const PeerGather& pg, cudaStream_t st)
{
    if (h_out == h_in || (d & 31) != 0 || pg.tp_size > 8) {
        return cudaErrorInvalidValue;
    }
    if (pg.tp_size > 1 && add && d <= NORM_CLUSTER * NORM_MAXJ * 256) {
        return launch_pdl_cluster(resid_rmsnorm_pack_tp_kernel, dim3(NORM_CLUSTER), dim3(256), NORM_CLUSTER, st, h_in, add, w,
                                  eps, d, packed, h_out, pg);
    }
    if (pg.tp_size > 1 && add) {
        return launch_pdl(resid_rmsnorm_pack_kernel<true>, dim3((d + 255) / 256), dim3(256), 0, st, h_in, add, w, eps, d,
                          packed, h_out, pg);
    }
    return launch_pdl(resid_rmsnorm_pack_kernel<false>, dim3((d + 255) / 256), dim3(256), 0, st, h_in, add, w, eps, d,
                      packed, h_out, pg);
}

cudaError_t ll_rope_kv(float* qkv, const int* pos, int pos_add, int rows, int n_heads, int n_kv, int hd, int rope_dim,
                       const float* rope_cos, const float* rope_sin, int max_seq, __half* cache_k, __half* cache_v,
                       cudaStream_t st)
{
    const int row_stride = (n_heads + 2 * n_kv) * hd;
    const int work = (n_heads + n_kv) * hd / 2 + n_kv * hd;
    return launch_pdl(rope_kv_kernel, dim3((work + 255) / 256, rows), dim3(256), 0, st, qkv, pos, pos_add, n_heads,
                      n_kv, hd, rope_dim, rope_cos, rope_sin, max_seq, cache_k, cache_v, row_stride);
}

cudaError_t ll_attn_fused(const float* qkv, const int* pos, int n_heads, int n_kv, int hd, int rope_dim,
                          const float* rope_cos, const float* rope_sin, int max_seq, __half* cache_k, __half* cache_v,
                          uint8_t* packed, cudaStream_t st)
{
    const int chunks = (n_heads * hd + 255) / 256;
    const dim3 grid(chunks * ATTN_CLUSTER), block(256);
    switch (hd) {
    case 64:
        return launch_pdl_cluster(attn_fused_kernel<2>, grid, block, ATTN_CLUSTER, st, qkv, pos, n_heads, n_kv, rope_dim,
                                  rope_cos, rope_sin, max_seq, cache_k, cache_v, packed);
    case 128:
        return launch_pdl_cluster(attn_fused_kernel<4>, grid, block, ATTN_CLUSTER, st, qkv, pos, n_heads, n_kv, rope_dim,
                                  rope_cos, rope_sin, max_seq, cache_k, cache_v, packed);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t ll_silu_mul_pack(const float* gu, int ffn, uint8_t* packed, cudaStream_t st)
{
    return launch_pdl(silu_mul_pack_kernel, dim3((ffn + 255) / 256), dim3(32), 0, st, gu, ffn, packed);
}

cudaError_t ll_argmax(const float* logits, int n, int index_offset, int ctas, int* best_pair, cudaStream_t st)
{
    return launch_pdl(argmax_kernel, dim3(ctas), dim3(1024), 0, st, logits, n, index_offset, best_pair);
}

cudaError_t ll_commit_token(const int* pairs, int ranks, int* token, int* pos, int* out_tokens, int* out_count,
                            cudaStream_t st)
{
    return launch_pdl(commit_token_kernel, dim3(1), dim3(32), 0, st, pairs, ranks, token, pos, out_tokens, out_count);
}

cudaError_t ll_resid_rmsnorm_rows(float* h, const float* add, const float* w, float eps, int d, int64_t m,
                                  __nv_bfloat16* xn, cudaStream_t st)
{
    resid_rmsnorm_rows_kernel<<<(unsigned)m, 256, 0, st>>>(h, add, w, eps, d, xn);
    return cudaGetLastError();
}

cudaError_t ll_attn_prefill(const float* qkv, int m, int pos0, int n_heads, int n_kv, int hd, int max_seq,
                            const __half* cache_k, const __half* cache_v, __nv_bfloat16* ctx, cudaStream_t st)
{
    const int row_stride = (n_heads + 2 * n_kv) * hd;
    const int64_t warps = (int64_t)m * n_heads;
    attn_prefill_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(qkv, row_stride, m, pos0, n_heads, n_kv, hd,
                                                                    max_seq, cache_k, cache_v, ctx);
    return cudaGetLastError();
}

cudaError_t ll_silu_mul_rows(const float* gu, int64_t m, int ffn, __nv_bfloat16* act, cudaStream_t st)
{
    silu_mul_rows_kernel<<<1024, 256, 0, st>>>(gu, m, ffn, act);
    return cudaGetLastError();
}

cudaError_t ll_add_rows(float* h, const float* add, int64_t total, cudaStream_t st)
{
    add_rows_kernel<<<1024, 256, 0, st>>>(h, add, total);
    return cudaGetLastError();
}

}  // namespace qmm

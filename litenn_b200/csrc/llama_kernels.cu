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
#include <algorithm>

#include <cuda_bf16.h>
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include "llama_device.cuh"
#include "llama_kernels.h"
#include "qmm_layout.cuh"
#include "qmm_pack.cuh"

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
    const int elems = block_elems(fmt), bytes = block_bytes(fmt);
    const int64_t row_bytes = (int64_t)(d / elems) * bytes;
    for (int r = blockIdx.y; r < n_rows; r += gridDim.y) {
        const uint8_t* row = raw + (int64_t)tokens[r] * row_bytes;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < d; i += gridDim.x * blockDim.x) {
            h[(int64_t)r * d + i] = dequant_raw_element(fmt, row + (i / elems) * bytes, i % elems);
        }
    }
}

__device__ __forceinline__ double warp_sum_double(double v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    }
    return v;
}

// What every producer of a matvec input leaves behind for element e of the residual stream `hv`:
// the stream itself, hv * w as the packed activations of the matvec that follows the RMSNorm,
// and the 32-block's sum of squares (the consumer applies 1/rms to its row sums).  One warp per
// 32-block, one element per lane.
__device__ __forceinline__ void emit_block32(float hv, int group, int e, const float* __restrict__ w,
                                             float* __restrict__ h_out, uint8_t* __restrict__ packed,
                                             double* __restrict__ ss_out)
{
    if (h_out) {
        h_out[e] = hv;
    }
    const double sq = warp_sum_double((double)hv * (double)hv);
    if ((threadIdx.x & 31) == 0) {
        ss_out[group] = sq;
    }
    warp_pack_block32(hv * w[e], packed + (size_t)(group >> 3) * XPK1_REC, group & 7);
}

// First kernel of a decoded token: the embedding row of *token becomes the residual stream, and
// the first block's attention-norm input is packed.  It waits for the previous token's last
// kernel BEFORE it lets its own dependents launch: that kernel sets the token and advances the
// position, which every later kernel of this token may read as soon as it starts.
__global__ void __launch_bounds__(128) embed_pack_kernel(int fmt, const uint8_t* __restrict__ raw,
                                                         const int* __restrict__ token, int d,
                                                         const float* __restrict__ w, float* __restrict__ h,
                                                         uint8_t* __restrict__ packed, double* __restrict__ ss_out)
{
    pdl_sync();
    pdl_trigger();
    const int group = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int e = group * 32 + (threadIdx.x & 31);
    if (group * 32 >= d) {
        return;
    }
    const int elems = block_elems(fmt), bytes = block_bytes(fmt);
    const uint8_t* row = raw + (int64_t)(*token) * (int64_t)(d / elems) * bytes;
    const float hv = dequant_raw_element(fmt, row + (e / elems) * bytes, e % elems);
    emit_block32(hv, group, e, w, h, packed, ss_out);
}

__device__ __forceinline__ uint2 ld_sys_v2(const uint2* p)
{
    uint2 q;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(q.x), "=r"(q.y) : "l"(p) : "memory");
    return q;
}

__device__ __forceinline__ void st_sys_v2(uint2* p, uint32_t a, uint32_t b)
{
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// hv = h_in + add (add optional), then emit_block32.  The stand-alone form of the matvec's
// EPI_RESID_PACK epilogue, for the places where the addend is not one matvec's row sums:
//   - tensor parallelism (TP): `add` is only this rank's addend; the other ranks' addends arrive
//     in pg.recv as {value, exchange number} packets stored by their matvec kernels (PeerScatter,
//     qmm_common.cuh).  A lane requests the packets of all peers at once, polls the ones that
//     have not arrived (bounded), and adds the addends in rank order, so every rank computes
//     bit-identical sums without a collective launch;
//   - the last row of a prefill, whose addend comes from the GEMM path.
// h_out may equal h_in (each element is touched by one lane only).
template <bool TP>
__global__ void __launch_bounds__(128) resid_pack_kernel(const float* __restrict__ h_in, const float* __restrict__ add,
                                                         const float* __restrict__ w, int d, float* __restrict__ h_out,
                                                         uint8_t* __restrict__ packed, double* __restrict__ ss_out,
                                                         PeerGather pg)
{
    pdl_trigger();
    // the position was advanced by the previous token's last kernel, which completed before this
    // token's first kernel let anything else launch (embed_pack_kernel)
    unsigned int epoch = 0;
    if (TP) {
        epoch = (unsigned int)(*pg.pos * pg.sites + pg.site + 1);
    }
    pdl_sync();
    const int group = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int e = group * 32 + (threadIdx.x & 31);
    if (group * 32 >= d) {
        return;
    }
    float a = 0.0f;
    if (TP) {
        constexpr int MAXR = 8;
        bool ok = *reinterpret_cast<volatile int*>(pg.status) == 0;  // after one timeout nothing waits again
        uint2 pk[MAXR];
#pragma unroll
        for (int r = 0; r < MAXR; ++r) {
            if (r < pg.tp_size && r != pg.tp_rank) {
                pk[r] = ld_sys_v2(pg.recv + (size_t)r * d + e);
            }
        }
        const float own = add[e];
#pragma unroll
        for (int r = 0; r < MAXR; ++r) {
            if (r < pg.tp_size) {
                if (r == pg.tp_rank) {
                    a += own;
                } else {
                    unsigned int spin = 0;
                    while (ok && pk[r].y != epoch) {
                        if (++spin > pg.spin_limit) {
                            ok = false;
                            atomicExch(pg.status, 5);  // a peer's addend never came; the sum is incomplete
                            break;
                        }
                        pk[r] = ld_sys_v2(pg.recv + (size_t)r * d + e);
                    }
                    a += __uint_as_float(pk[r].x);
                }
            }
        }
    } else if (add) {
        a = add[e];
    }
    emit_block32(h_in[e] + a, group, e, w, h_out, packed, ss_out);
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

// CTAs per 256-wide context chunk = key splits / 4.  One sequence wants the most splits a portable cluster
// allows (cluster sizes 4 and 16 measured slower than 8: 39.2 / 38.1 / 36.6 us per block of the 7B shape); a
// batch of sequences already fills the SMs with (sequence, chunk) pairs, and fewer, longer splits keep its
// CTAs in one wave.
constexpr int attn_cluster_for(int batch)
{
    return batch >= 8 ? 2 : batch >= 3 ? 4 : 8;
}

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
template <int DPL, int ATTN_CLUSTER>  // head dims per lane = hd / 32 (2 or 4); CTAs per 256-wide context chunk
__global__ void __launch_bounds__(256) attn_fused_kernel(const float* __restrict__ qkv, const int* __restrict__ pos_ptr,
                                                         int n_heads, int n_kv, int rope_dim,
                                                         const float* __restrict__ rope_cos,
                                                         const float* __restrict__ rope_sin, int max_seq,
                                                         __half* __restrict__ cache_k, __half* __restrict__ cache_v,
                                                         uint8_t* __restrict__ packed, AttnBatch ab)
{
    constexpr int hd = 32 * DPL;
    // batched decode: blockIdx.y is the sequence; each has its own qkv row, position and cache
    qkv += (int64_t)blockIdx.y * ab.qkv_stride;
    pos_ptr += blockIdx.y;
    cache_k += (int64_t)blockIdx.y * ab.cache_stride;
    cache_v += (int64_t)blockIdx.y * ab.cache_stride;
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
        if (ab.ctx) {  // batched decode keeps fp32 rows; the rows are packed together afterwards
            if (chunk * 256 + (int)threadIdx.x < n_heads * hd) {
                ab.ctx[(int64_t)blockIdx.y * ab.ctx_stride + chunk * 256 + threadIdx.x] = vals[threadIdx.x];
            }
            return;
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        float r8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r8[i] = vals[8 * threadIdx.x + i];
        }
        warp_pack_chunk(r8, packed + (size_t)chunk * XPK1_REC);
    }
}

// Greedy argmax, first stage (lowest index wins ties): CTA b writes its (value bits, index)
// candidate to best_pair[2b..2b+1].
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int n, int index_offset,
                                                      int* __restrict__ best_pair, int64_t row_stride)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_sync();
    logits += (int64_t)blockIdx.y * row_stride;  // batched decode: one row of logits per sequence
    best_pair += (int64_t)blockIdx.y * 2 * gridDim.x;
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

// Picks the winner among this rank's `n_local` (value, index) candidates, and with tensor
// parallelism among the ranks' winners: every rank stores its winner as two packets
// {value bits, number} {index, number} into each peer's buffer (number = position + 1) and polls
// the peers' packets (bounded).  Ties go to the lowest index, so all ranks agree.  Then stores
// the token and advances the position.  One warp.
__global__ void __launch_bounds__(32) commit_token_kernel(const int* __restrict__ pairs, int n_local, ArgmaxExchange ax,
                                                          int* __restrict__ token, int* __restrict__ pos,
                                                          int* __restrict__ out_tokens, int* __restrict__ out_count,
                                                          TokenReport report)
{
    pdl_trigger();
    pdl_sync();
    const int lane = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = lane; i < n_local; i += 32) {
        const float v = __int_as_float(pairs[2 * i]);
        const int ix = pairs[2 * i + 1];
        if (v > bv || (v == bv && ix < bi)) {
            bv = v;
            bi = ix;
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
    if (ax.tp_size > 1) {
        const unsigned int number = (unsigned int)(*pos + 1);
        if (lane < ax.tp_size && lane != ax.tp_rank) {
            uint2* dst = ax.peer[lane] + 2 * ax.tp_rank;
            st_sys_v2(dst, __float_as_uint(bv), number);
            st_sys_v2(dst + 1, (uint32_t)bi, number);
        }
        float cv = -INFINITY;
        int ci = 0x7FFFFFFF;
        if (lane == ax.tp_rank) {
            cv = bv;
            ci = bi;
        } else if (lane < ax.tp_size) {
            bool ok = *reinterpret_cast<volatile int*>(ax.status) == 0;
            const uint2* src = ax.recv + 2 * lane;
            uint2 a = ld_sys_v2(src), b = ld_sys_v2(src + 1);
            unsigned int spin = 0;
            while (ok && (a.y != number || b.y != number)) {
                if (++spin > ax.spin_limit) {
                    ok = false;
                    atomicExch(ax.status, 6);  // a peer's arg-max candidate never came
                    break;
                }
                a = ld_sys_v2(src);
                b = ld_sys_v2(src + 1);
            }
            if (ok) {
                cv = __uint_as_float(a.x);
                ci = (int)b.x;
            }
        }
        bv = cv;
        bi = ci;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
    }
    if (lane == 0) {
        *token = bi;
        out_tokens[*out_count] = bi;
        *out_count += 1;
        *pos += 1;
        if (report.host) {
            // the token and the two status words in host-visible memory: a caller that takes one token at a
            // time reads them after the stream has drained, without a copy of its own
            report.host[0] = bi;
            report.host[1] = *reinterpret_cast<const volatile int*>(report.model_status);
            report.host[2] = *reinterpret_cast<const volatile int*>(report.library_status);
        }
    }
}

// Batched decode: one warp per sequence picks the winner among the ranks' candidates of its row
// (pairs[rank][row][2 * per_rank]; lowest index wins ties), stores the row's next token, appends it to
// the step-major output list and advances the row's position.
__global__ void __launch_bounds__(512) commit_batch_kernel(const int* __restrict__ pairs, int per_rank, int ranks,
                                                           int batch, int* __restrict__ tokens, int* __restrict__ pos,
                                                           int* __restrict__ out_tokens, int* __restrict__ out_steps)
{
    pdl_trigger();
    pdl_sync();
    const int lane = threadIdx.x & 31, row = threadIdx.x >> 5;
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    if (row < batch) {
        for (int i = lane; i < per_rank * ranks; i += 32) {
            const int r = i / per_rank, c = i % per_rank;
            const int* p = pairs + ((int64_t)r * batch + row) * 2 * per_rank + 2 * c;
            const float v = __int_as_float(p[0]);
            const int ix = p[1];
            if (v > bv || (v == bv && ix < bi)) {
                bv = v;
                bi = ix;
            }
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
    const int step = *out_steps;
    __syncthreads();  // every warp has read the step count before it moves
    if (row < batch && lane == 0) {
        tokens[row] = bi;
        out_tokens[(int64_t)step * batch + row] = bi;
        pos[row] += 1;
    }
    if (threadIdx.x == 0) {
        *out_steps = step + 1;
    }
}

// ---- prefill (many tokens) ------------------------------------------------------------------------

__device__ __forceinline__ void store_row_value(__nv_bfloat16* p, float v)
{
    *p = __float2bfloat16_rn(v);
}
__device__ __forceinline__ void store_row_value(float* p, float v)
{
    *p = v;
}

__device__ __forceinline__ void store_row_values(__nv_bfloat16* p, float a, float b, float c, float d4)
{
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d4);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}
__device__ __forceinline__ void store_row_values(float* p, float a, float b, float c, float d4)
{
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d4);
}

// Per row: h += add (optional); xn = rmsnorm(h) * w, as bf16 for the GEMM or as fp32 for the packed matvec.
// One CTA per row (d a multiple of 4); a thread keeps its float4 pieces of the row in registers between the
// two passes (up to 8 pieces = d <= 8192 with 256 threads; longer rows re-read h), and all of a pass's loads
// are issued before the first is used: with scalar loads in a 16-trip loop the kernel took 18 us for 16 rows.
// Statistics and the scale by the weight in double, one cast (ComputePrimitives.h:755-816); one double
// reciprocal per row instead of a division per element (within one unit in the last place of the double
// quotient, so the fp32 result is the reference's).
template <typename OutT>
__global__ void __launch_bounds__(256) resid_rmsnorm_rows_kernel(float* __restrict__ h, const float* __restrict__ add,
                                                                 const float* __restrict__ w, float eps, int d,
                                                                 OutT* __restrict__ xn)
{
    constexpr int KEEP = 8;
    __shared__ double red[32];
    const int64_t row = blockIdx.x;
    float4* hr = reinterpret_cast<float4*>(h + row * d);
    const float4* ar = add ? reinterpret_cast<const float4*>(add + row * d) : nullptr;
    const int n4 = d >> 2;
    float4 keep[KEEP];
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const int i = threadIdx.x + j * 256;
        keep[j] = i < n4 ? hr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (ar) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < n4) {
                const float4 a = ar[i];
                keep[j].x += a.x;
                keep[j].y += a.y;
                keep[j].z += a.z;
                keep[j].w += a.w;
                hr[i] = keep[j];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        ss += (double)keep[j].x * (double)keep[j].x + (double)keep[j].y * (double)keep[j].y +
              (double)keep[j].z * (double)keep[j].z + (double)keep[j].w * (double)keep[j].w;
    }
    for (int i = threadIdx.x + KEEP * 256; i < n4; i += 256) {  // rows longer than 8192
        float4 v = hr[i];
        if (ar) {
            const float4 a = ar[i];
            v = make_float4(v.x + a.x, v.y + a.y, v.z + a.z, v.w + a.w);
            hr[i] = v;
        }
        ss += (double)v.x * (double)v.x + (double)v.y * (double)v.y + (double)v.z * (double)v.z + (double)v.w * (double)v.w;
    }
    ss = block_sum_double(ss, red);
    const double inv = 1.0 / sqrt(ss / (double)d + (double)eps);
    const float4* wr = reinterpret_cast<const float4*>(w);
    auto emit = [&](int i, const float4& v) {
        const float4 ww = wr[i];
        store_row_values(xn + row * d + 4 * (int64_t)i, (float)(((double)v.x * inv) * (double)ww.x),
                         (float)(((double)v.y * inv) * (double)ww.y), (float)(((double)v.z * inv) * (double)ww.z),
                         (float)(((double)v.w * inv) * (double)ww.w));
    };
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            emit(i, keep[j]);
        }
    }
    for (int i = threadIdx.x + KEEP * 256; i < n4; i += 256) {
        emit(i, hr[i]);
    }
}

// Causal attention over the fp16 cache for rows 0..m-1 at positions pos0+row.  The kernel is bound by the L2
// reads of K and V (every row streams the whole prefix of its head), so one warp serves ROWS consecutive rows of
// one head and reuses each loaded batch of eight keys for all of them; a row simply ignores the keys beyond its
// own position.  Online softmax per row, one rescale per batch; output bf16 ctx[m][n_heads*hd].
template <int DPL, int ROWS>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const float* __restrict__ qkv, int row_stride, int m,
                                                           int pos0, int n_heads, int n_kv, int max_seq,
                                                           const __half* __restrict__ cache_k,
                                                           const __half* __restrict__ cache_v,
                                                           __nv_bfloat16* __restrict__ ctx)
{
    constexpr int hd = 32 * DPL;
    const int lane = threadIdx.x & 31;
    const int groups = (m + ROWS - 1) / ROWS;
    const int64_t wid = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wid >= (int64_t)groups * n_heads) {
        return;
    }
    // the longest rows first: the last CTAs to start are the shortest
    const int row0 = (groups - 1 - (int)(wid / n_heads)) * ROWS, head = (int)(wid % n_heads);
    const int kvh = head / (n_heads / n_kv);
    const float scale = rsqrtf((float)hd);
    float qv[ROWS][DPL], acc[ROWS][DPL], mx[ROWS], l[ROWS];
    int keys[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int row = min(row0 + r, m - 1);  // a ragged last group repeats the last row (stored once)
        keys[r] = pos0 + row + 1;
        mx[r] = -INFINITY;
        l[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            qv[r][i] = qkv[(int64_t)row * row_stride + head * hd + lane * DPL + i] * scale;
            acc[r][i] = 0.0f;
        }
    }
    const __half* kb = cache_k + (int64_t)kvh * max_seq * hd + lane * DPL;
    const __half* vb = cache_v + (int64_t)kvh * max_seq * hd + lane * DPL;
    const int n_keys = keys[ROWS - 1];
    KvBatch<DPL> a, b;
    kv_batch_load<DPL>(a, kb, vb, 0, n_keys);
    for (int kbase = 0; kbase < n_keys; kbase += 16) {
        if (kbase + 8 < n_keys) {
            kv_batch_load<DPL>(b, kb, vb, kbase + 8, n_keys);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            kv_batch_apply<DPL>(a, qv[r], kbase, keys[r], mx[r], l[r], acc[r]);
        }
        if (kbase + 16 < n_keys) {
            kv_batch_load<DPL>(a, kb, vb, kbase + 16, n_keys);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            kv_batch_apply<DPL>(b, qv[r], kbase + 8, keys[r], mx[r], l[r], acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        if (row0 + r < m) {
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                ctx[(int64_t)(row0 + r) * n_heads * hd + head * hd + lane * DPL + i] =
                    __float2bfloat16_rn(acc[r][i] / l[r]);
            }
        }
    }
}

// act[m][ffn] = bf16(silu(gate) * up) from gu[m][2*ffn], whose columns are the gate|up weight's rows:
// groups of 8 gate channels followed by the same 8 channels of up (the matvec's SwiGLU epilogue
// wants both halves of a channel in one 16-row tile).
template <typename OutT>
__global__ void silu_mul_rows_kernel(const float* __restrict__ gu, int64_t m, int ffn, OutT* __restrict__ act)
{
    const int64_t total = m * ffn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / ffn;
        const int c = (int)(i % ffn);
        const int col = (c >> 3) * 16 + (c & 7);
        const float g = gu[r * 2 * ffn + col], u = gu[r * 2 * ffn + col + 8];
        store_row_value(&act[i], (g * (1.0f / (1.0f + expf(-g)))) * u);
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
    embed_row_kernel<<<dim3((d + 255) / 256, n_rows < 1024 ? n_rows : 1024), 256, 0, st>>>(fmt, raw, tokens, n_rows, d, h);
    return cudaGetLastError();
}

cudaError_t ll_embed_pack(int fmt, const uint8_t* raw, const int* token, int d, const float* w, float* h,
                          uint8_t* packed, double* ss_out, cudaStream_t st)
{
    if ((d & 31) != 0) {
        return cudaErrorInvalidValue;
    }
    return launch_pdl(embed_pack_kernel, dim3((d / 32 + 3) / 4), dim3(128), 0, st, fmt, raw, token, d, w, h, packed, ss_out);
}

cudaError_t ll_resid_pack(const float* h_in, const float* add, const float* w, int d, float* h_out, uint8_t* packed,
                          double* ss_out, const PeerGather& pg, cudaStream_t st)
{
    if ((d & 31) != 0 || pg.tp_size > 8) {
        return cudaErrorInvalidValue;
    }
    const dim3 grid((d / 32 + 3) / 4), block(128);
    if (pg.tp_size > 1) {
        if (!add) {
            return cudaErrorInvalidValue;
        }
        return launch_pdl(resid_pack_kernel<true>, grid, block, 0, st, h_in, add, w, d, h_out, packed, ss_out, pg);
    }
    return launch_pdl(resid_pack_kernel<false>, grid, block, 0, st, h_in, add, w, d, h_out, packed, ss_out, pg);
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
                          uint8_t* packed, int batch, const AttnBatch& ab, cudaStream_t st)
{
    const int chunks = (n_heads * hd + 255) / 256;
    const int cl = attn_cluster_for(batch);
    const dim3 grid(chunks * cl, batch), block(256);
#define QMM_ATTN_LAUNCH(DPL, CL)                                                                                         \
    return launch_pdl_cluster(attn_fused_kernel<DPL, CL>, grid, block, CL, st, qkv, pos, n_heads, n_kv, rope_dim, rope_cos, \
                              rope_sin, max_seq, cache_k, cache_v, packed, ab)
    if (hd == 64) {
        if (cl == 2) { QMM_ATTN_LAUNCH(2, 2); }
        if (cl == 4) { QMM_ATTN_LAUNCH(2, 4); }
        QMM_ATTN_LAUNCH(2, 8);
    }
    if (hd == 128) {
        if (cl == 2) { QMM_ATTN_LAUNCH(4, 2); }
        if (cl == 4) { QMM_ATTN_LAUNCH(4, 4); }
        QMM_ATTN_LAUNCH(4, 8);
    }
#undef QMM_ATTN_LAUNCH
    return cudaErrorInvalidValue;
}

cudaError_t ll_argmax(const float* logits, int n, int index_offset, int ctas, int* best_pair, int rows,
                      int64_t row_stride, cudaStream_t st)
{
    return launch_pdl(argmax_kernel, dim3(ctas, rows), dim3(1024), 0, st, logits, n, index_offset, best_pair, row_stride);
}

cudaError_t ll_commit_batch(const int* pairs, int per_rank, int ranks, int batch, int* tokens, int* pos, int* out_tokens,
                            int* out_steps, cudaStream_t st)
{
    if (batch < 1 || batch > 16) {
        return cudaErrorInvalidValue;
    }
    return launch_pdl(commit_batch_kernel, dim3(1), dim3(32 * batch), 0, st, pairs, per_rank, ranks, batch, tokens, pos,
                      out_tokens, out_steps);
}

cudaError_t ll_commit_token(const int* pairs, int n_local, const ArgmaxExchange& ax, int* token, int* pos,
                            int* out_tokens, int* out_count, const TokenReport& report, cudaStream_t st)
{
    if (ax.tp_size > 8) {
        return cudaErrorInvalidValue;
    }
    return launch_pdl(commit_token_kernel, dim3(1), dim3(32), 0, st, pairs, n_local, ax, token, pos, out_tokens, out_count,
                      report);
}

cudaError_t ll_resid_rmsnorm_rows(float* h, const float* add, const float* w, float eps, int d, int64_t m,
                                  __nv_bfloat16* xn, cudaStream_t st)
{
    resid_rmsnorm_rows_kernel<__nv_bfloat16><<<(unsigned)m, 256, 0, st>>>(h, add, w, eps, d, xn);
    return cudaGetLastError();
}

cudaError_t ll_resid_rmsnorm_rows_f32(float* h, const float* add, const float* w, float eps, int d, int64_t m, float* xn,
                                      cudaStream_t st)
{
    resid_rmsnorm_rows_kernel<float><<<(unsigned)m, 256, 0, st>>>(h, add, w, eps, d, xn);
    return cudaGetLastError();
}

cudaError_t ll_attn_prefill(const float* qkv, int m, int pos0, int n_heads, int n_kv, int hd, int max_seq,
                            const __half* cache_k, const __half* cache_v, __nv_bfloat16* ctx, cudaStream_t st)
{
    constexpr int ROWS = 4;
    const int row_stride = (n_heads + 2 * n_kv) * hd;
    const int64_t warps = (int64_t)((m + ROWS - 1) / ROWS) * n_heads;
    const unsigned grid = (unsigned)((warps + 3) / 4);
    switch (hd) {
    case 64:
        attn_prefill_kernel<2, ROWS><<<grid, 128, 0, st>>>(qkv, row_stride, m, pos0, n_heads, n_kv, max_seq, cache_k,
                                                           cache_v, ctx);
        break;
    case 128:
        attn_prefill_kernel<4, ROWS><<<grid, 128, 0, st>>>(qkv, row_stride, m, pos0, n_heads, n_kv, max_seq, cache_k,
                                                           cache_v, ctx);
        break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t ll_silu_mul_rows(const float* gu, int64_t m, int ffn, __nv_bfloat16* act, cudaStream_t st)
{
    silu_mul_rows_kernel<__nv_bfloat16><<<1024, 256, 0, st>>>(gu, m, ffn, act);
    return cudaGetLastError();
}

cudaError_t ll_silu_mul_rows_f32(const float* gu, int64_t m, int ffn, float* act, cudaStream_t st)
{
    silu_mul_rows_kernel<float><<<(unsigned)std::min<int64_t>(1024, (m * ffn + 255) / 256), 256, 0, st>>>(gu, m, ffn, act);
    return cudaGetLastError();
}

cudaError_t ll_add_rows(float* h, const float* add, int64_t total, cudaStream_t st)
{
    add_rows_kernel<<<1024, 256, 0, st>>>(h, add, total);
    return cudaGetLastError();
}

}  // namespace qmm

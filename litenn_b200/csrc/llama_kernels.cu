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
#include <cuda_fp16.h>

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

// Quantize the 256 values a warp holds (lane L: positions 8L..8L+7 of chunk c) and write the
// compact batch-1 packed form (qmm_common.cuh: xq [kc][8][8] uint2, xs [kc], xsum [kc][8] int2).
__device__ __forceinline__ void warp_pack_chunk(const float (&v)[8], int c, int kc, uint8_t* out)
{
    const int lane = threadIdx.x & 31;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    }
    const float inv = amax > 0.0f ? 32639.0f / amax : 0.0f;
    uint32_t hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
    int bsum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int q = __float2int_rn(v[i] * inv);
        q = max(-32639, min(32639, q));
        bsum += q;
        const int l = ((q + 128) & 0xFF) - 128;
        const int h = (q - l) >> 8;
        hi[i >> 2] |= (uint32_t)(h & 0xFF) << (8 * (i & 3));
        lo[i >> 2] |= (uint32_t)(l & 0xFF) << (8 * (i & 3));
    }
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 1);
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 2);
    // positions 8*part..8*part+7 of block b: fragment lanes t = 2*(part&1) and +1, word part>>1
    const int b = lane >> 2, part = lane & 3;
    uint32_t* xq = reinterpret_cast<uint32_t*>(out) + ((size_t)(c * 8 + b) * 8) * 2;
    const int t0 = 2 * (part & 1), word = part >> 1;
    xq[((0 * 4 + t0) * 2) + word] = hi[0];
    xq[((0 * 4 + t0 + 1) * 2) + word] = hi[1];
    xq[((1 * 4 + t0) * 2) + word] = lo[0];
    xq[((1 * 4 + t0 + 1) * 2) + word] = lo[1];
    if (lane == 0) {
        reinterpret_cast<float*>(out + xpack1_xs_offset(kc))[c] = amax / 32639.0f;
    }
    if (part == 0) {
        reinterpret_cast<int2*>(out + xpack1_xsum_offset(kc))[c * 8 + b] = make_int2(8 * bsum, 128 * bsum);
    }
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

// One CTA: h += add (optional); xn = rmsnorm(h) * w; packed = pack(xn).  Also the place where
// the decode position advances (bump_pos) so that a replayed graph needs no host input.
__global__ void __launch_bounds__(1024) resid_rmsnorm_pack_kernel(float* __restrict__ h, const float* __restrict__ add,
                                                                  const float* __restrict__ w, float eps, int d,
                                                                  uint8_t* __restrict__ packed,
                                                                  float* __restrict__ xn_out)
{
    __shared__ double red[32];
    extern __shared__ float xs_buf[];  // d floats
    pdl_trigger();
    pdl_sync();
    double ss = 0.0;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = h[i];
        if (add) {
            v += add[i];
            h[i] = v;
        }
        xs_buf[i] = v;
        ss += (double)v * (double)v;
    }
    ss = block_sum_double(ss, red);
    const double inv = 1.0 / sqrt(ss / (double)d + (double)eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = (float)((double)xs_buf[i] * inv) * w[i];
        xs_buf[i] = v;
        if (xn_out) {
            xn_out[i] = v;
        }
    }
    __syncthreads();
    if (packed) {
        const int kc = (d + 255) / 256;
        const int lane = threadIdx.x & 31;
        for (int c = threadIdx.x >> 5; c < kc; c += blockDim.x >> 5) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int idx = c * 256 + 8 * lane + i;
                v[i] = idx < d ? xs_buf[idx] : 0.0f;
            }
            warp_pack_chunk(v, c, kc, packed);
        }
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

// Decode attention, split over the cached positions: grid (n_heads, splits), 128 threads.
// Each warp takes batches of 8 keys (all loads of a batch are issued before any use), keeps an
// online softmax, and the four warps' partials (max, sum, acc[hd]) are merged into `part`.
template <int DPL>  // head dims per lane = hd / 32 (2, 4 or 8)
__global__ void __launch_bounds__(128) attn_decode_kernel(const float* __restrict__ q, const int* __restrict__ pos_ptr,
                                                          int n_heads, int n_kv, int max_seq,
                                                          const __half* __restrict__ cache_k,
                                                          const __half* __restrict__ cache_v, float* __restrict__ part)
{
    constexpr int hd = 32 * DPL;
    __shared__ float sm[4][hd + 2];
    pdl_trigger();
    pdl_sync();
    const int head = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int kvh = head / (n_heads / n_kv);
    const int n_keys = *pos_ptr + 1;
    const int per = (n_keys + splits - 1) / splits;
    const int k0 = split * per, k1 = min(n_keys, k0 + per);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float scale = rsqrtf((float)hd);
    float qv[DPL], acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        qv[i] = q[head * hd + lane * DPL + i] * scale;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const __half* kb = cache_k + (int64_t)kvh * max_seq * hd + lane * DPL;
    const __half* vb = cache_v + (int64_t)kvh * max_seq * hd + lane * DPL;
    for (int kbase = k0 + warp * 8; kbase < k1; kbase += 32) {
        __half kr[8][DPL], vr[8][DPL];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = min(kbase + j, k1 - 1);
#pragma unroll
            for (int i = 0; i < DPL; i += 2) {
                *reinterpret_cast<__half2*>(&kr[j][i]) = *reinterpret_cast<const __half2*>(kb + (int64_t)k * hd + i);
                *reinterpret_cast<__half2*>(&vr[j][i]) = *reinterpret_cast<const __half2*>(vb + (int64_t)k * hd + i);
            }
        }
        float sc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                dot += qv[i] * __half2float(kr[j][i]);
            }
            sc[j] = dot;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sc[j] += __shfl_xor_sync(0xFFFFFFFFu, sc[j], o);
            }
        }
        float mb = m;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (kbase + j < k1) {
                mb = fmaxf(mb, sc[j]);
            }
        }
        const float corr = __expf(m - mb);
        l *= corr;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            acc[i] *= corr;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (kbase + j < k1) {
                const float p = __expf(sc[j] - mb);
                l += p;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    acc[i] += p * __half2float(vr[j][i]);
                }
            }
        }
        m = mb;
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
    float M = -INFINITY;
    for (int w = 0; w < 4; ++w) {
        M = fmaxf(M, sm[w][hd]);
    }
    float* out = part + ((int64_t)head * splits + split) * (hd + 2);
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        float a = 0.0f;
        for (int w = 0; w < 4; ++w) {
            const float mw = sm[w][hd];
            a += mw == -INFINITY ? 0.0f : sm[w][i] * __expf(mw - M);
        }
        out[i] = a;
    }
    if (threadIdx.x == 0) {
        float L = 0.0f;
        for (int w = 0; w < 4; ++w) {
            const float mw = sm[w][hd];
            L += mw == -INFINITY ? 0.0f : sm[w][hd + 1] * __expf(mw - M);
        }
        out[hd] = M;
        out[hd + 1] = L;
    }
}

// Merge the split partials into the context vector and pack it: one CTA (256 threads) per
// 256-wide chunk of ctx[n_heads*hd] — the activation quantization is per chunk, so chunks
// are independent.
__global__ void __launch_bounds__(256) attn_combine_pack_kernel(const float* __restrict__ part, int n_heads, int hd,
                                                                int splits, uint8_t* __restrict__ packed,
                                                                float* __restrict__ ctx_out)
{
    __shared__ float wgt[8][64];   // up to 8 heads per chunk (hd >= 32), up to 64 splits
    __shared__ float vals[256];
    pdl_trigger();
    pdl_sync();
    const int d = n_heads * hd;
    const int c = blockIdx.x;
    const int kc = (d + 255) / 256;
    const int heads_here = 256 / hd;
    // per (head, split) weight exp(m_s - M) / L
    if (threadIdx.x < heads_here) {
        const int head = c * heads_here + threadIdx.x;
        if (head < n_heads) {
            const float* p = part + (int64_t)head * splits * (hd + 2);
            float M = -INFINITY;
            for (int s2 = 0; s2 < splits; ++s2) {
                M = fmaxf(M, p[s2 * (hd + 2) + hd]);
            }
            float L = 0.0f;
            for (int s2 = 0; s2 < splits; ++s2) {
                const float ms = p[s2 * (hd + 2) + hd];
                const float f = ms == -INFINITY ? 0.0f : __expf(ms - M);
                wgt[threadIdx.x][s2] = f;
                L += p[s2 * (hd + 2) + hd + 1] * f;
            }
            for (int s2 = 0; s2 < splits; ++s2) {
                wgt[threadIdx.x][s2] /= L;
            }
        }
    }
    __syncthreads();
    const int idx = c * 256 + threadIdx.x;
    float v = 0.0f;
    if (idx < d) {
        const int head = idx / hd, e = idx % hd;
        const float* p = part + (int64_t)head * splits * (hd + 2);
        for (int s2 = 0; s2 < splits; ++s2) {
            v += p[s2 * (hd + 2) + e] * wgt[head - c * heads_here][s2];
        }
        if (ctx_out) {
            ctx_out[idx] = v;
        }
    }
    vals[threadIdx.x] = v;
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

cudaError_t ll_resid_rmsnorm_pack(float* h, const float* add, const float* w, float eps, int d, uint8_t* packed,
                                  float* xn_out, cudaStream_t st)
{
    static bool configured = false;
    const size_t smem = (size_t)d * sizeof(float);
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(resid_rmsnorm_pack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             200 * 1024);
        if (e != cudaSuccess) {
            return e;
        }
        configured = true;
    }
    return launch_pdl(resid_rmsnorm_pack_kernel, dim3(1), dim3(1024), smem, st, h, add, w, eps, d, packed, xn_out);
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

cudaError_t ll_attn_decode(const float* q, const int* pos, int n_heads, int n_kv, int hd, int max_seq,
                           const __half* cache_k, const __half* cache_v, int splits, float* part, cudaStream_t st)
{
    const dim3 grid(n_heads, splits), block(128);
    switch (hd) {
    case 64: return launch_pdl(attn_decode_kernel<2>, grid, block, 0, st, q, pos, n_heads, n_kv, max_seq, cache_k, cache_v, part);
    case 128: return launch_pdl(attn_decode_kernel<4>, grid, block, 0, st, q, pos, n_heads, n_kv, max_seq, cache_k, cache_v, part);
    case 256: return launch_pdl(attn_decode_kernel<8>, grid, block, 0, st, q, pos, n_heads, n_kv, max_seq, cache_k, cache_v, part);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t ll_attn_combine_pack(const float* part, int n_heads, int hd, int splits, uint8_t* packed, float* ctx_out,
                                 cudaStream_t st)
{
    if (splits > 64 || 256 % hd != 0) {
        return cudaErrorInvalidValue;
    }
    const int d = n_heads * hd;
    return launch_pdl(attn_combine_pack_kernel, dim3((d + 255) / 256), dim3(256), 0, st, part, n_heads, hd, splits,
                      packed, ctx_out);
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

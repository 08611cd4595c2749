// Device-side pieces shared by the decoder's per-operator kernels (llama_kernels.cu) and the
// persistent decoder kernel (llama_mega.cu): activation packing for the batch-1 matvec and
// the online-softmax update over batches of cached keys.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "qmm_common.cuh"

namespace qmm {
namespace {

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

// Eight cached keys/values of one kv head, DPL dims per lane.
template <int DPL>
struct KvBatch {
    __half k[8][DPL], v[8][DPL];
};

template <int DPL>
__device__ __forceinline__ void kv_batch_load(KvBatch<DPL>& b, const __half* kb, const __half* vb, int kbase, int k1)
{
    constexpr int hd = 32 * DPL;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int k = max(0, min(kbase + j, k1 - 1));
#pragma unroll
        for (int i = 0; i < DPL; i += 2) {
            *reinterpret_cast<__half2*>(&b.k[j][i]) = *reinterpret_cast<const __half2*>(kb + (int64_t)k * hd + i);
            *reinterpret_cast<__half2*>(&b.v[j][i]) = *reinterpret_cast<const __half2*>(vb + (int64_t)k * hd + i);
        }
    }
}

// Online-softmax update with the keys kbase..kbase+7 (those < k1) of a loaded batch.
template <int DPL>
__device__ __forceinline__ void kv_batch_apply(const KvBatch<DPL>& b, const float (&qv)[DPL], int kbase, int k1,
                                               float& m, float& l, float (&acc)[DPL])
{
    if (kbase >= k1) {
        return;
    }
    float sc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            dot += qv[i] * __half2float(b.k[j][i]);
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
                acc[i] += p * __half2float(b.v[j][i]);
            }
        }
    }
    m = mb;
}

}  // namespace
}  // namespace qmm

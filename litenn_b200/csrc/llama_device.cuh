// Device-side pieces of the decoder's attention kernels (llama_kernels.cu): the online-softmax
// update over batches of cached keys.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "qmm_common.cuh"

namespace qmm {
namespace {

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

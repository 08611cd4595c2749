// Writers of the compact (batch 1) packed-activation records of qmm_common.cuh, for every
// kernel that produces the input of a matvec: the stand-alone pack kernel, the matvec's own
// fused epilogues, the embedding row kernel, decode attention and the tensor-parallel gather.
// A 32-wide block is quantized on its own (scale = max|x| / 32639), so a producer that owns
// 32 consecutive activations can write its block of the record without seeing the others.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "qmm_common.cuh"

namespace qmm {
namespace {

// 16-bit quantization of one value against its block's inverse scale, as two signed bytes.
__device__ __forceinline__ int quant16(float v, float inv, int& hi, int& lo)
{
    int q = __float2int_rn(v * inv);
    q = max(-32639, min(32639, q));  // keeps both signed digits inside int8
    lo = ((q + 128) & 0xFF) - 128;
    hi = (q - lo) >> 8;
    return q;
}

// One warp, lane i holding activation i of block `b` of the chunk whose record starts at `rec`.
__device__ __forceinline__ void warp_pack_block32(float v, uint8_t* rec, int b)
{
    const int lane = threadIdx.x & 31;
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    }
    const float inv = amax > 0.0f ? 32639.0f / amax : 0.0f;
    int hi, lo;
    int q = quant16(v, inv, hi, lo);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        q += __shfl_xor_sync(0xFFFFFFFFu, q, o);
    }
    // word (digit, t, half) = bytes of activations half*16 + 4t .. +3: gather them inside the quad
    uint32_t hw = (uint32_t)(hi & 0xFF) << (8 * (lane & 3));
    uint32_t lw = (uint32_t)(lo & 0xFF) << (8 * (lane & 3));
    hw |= __shfl_xor_sync(0xFFFFFFFFu, hw, 1);
    lw |= __shfl_xor_sync(0xFFFFFFFFu, lw, 1);
    hw |= __shfl_xor_sync(0xFFFFFFFFu, hw, 2);
    lw |= __shfl_xor_sync(0xFFFFFFFFu, lw, 2);
    uint32_t* xq = reinterpret_cast<uint32_t*>(rec + b * 64);
    if ((lane & 3) == 0) {
        const int quad = lane >> 2, half = quad >> 2, t = quad & 3;
        xq[(0 * 4 + t) * 2 + half] = hw;
        xq[(1 * 4 + t) * 2 + half] = lw;
    }
    if (lane == 0) {
        reinterpret_cast<int4*>(rec + XPK1_META)[b] = make_int4(8 * q, 128 * q, __float_as_int(amax / 32639.0f), 0);
    }
}

// One warp, lane L holding activations 4L..4L+3 of a 128-wide span = blocks b0..b0+3 of one record
// (b0 = 0 or 4): a lane's four values are exactly one fragment word per digit, so nothing has
// to be gathered; scale and sum go over the eight lanes of a block.
__device__ __forceinline__ void warp_pack_span128(const float4& v, uint8_t* rec, int b0)
{
    const int lane = threadIdx.x & 31;
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    }
    const float inv = amax > 0.0f ? 32639.0f / amax : 0.0f;
    int hi[4], lo[4];
    int q = quant16(v.x, inv, hi[0], lo[0]) + quant16(v.y, inv, hi[1], lo[1]) + quant16(v.z, inv, hi[2], lo[2]) +
            quant16(v.w, inv, hi[3], lo[3]);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        q += __shfl_xor_sync(0xFFFFFFFFu, q, o);
    }
    uint32_t hw = 0u, lw = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        hw |= (uint32_t)(hi[i] & 0xFF) << (8 * i);
        lw |= (uint32_t)(lo[i] & 0xFF) << (8 * i);
    }
    const int b = b0 + (lane >> 3), l8 = lane & 7, half = l8 >> 2, t = l8 & 3;
    uint32_t* xq = reinterpret_cast<uint32_t*>(rec + b * 64);
    xq[(0 * 4 + t) * 2 + half] = hw;
    xq[(1 * 4 + t) * 2 + half] = lw;
    if (l8 == 0) {
        reinterpret_cast<int4*>(rec + XPK1_META)[b] = make_int4(8 * q, 128 * q, __float_as_int(amax / 32639.0f), 0);
    }
}

// One warp, lane L holding activations 8L..8L+7 of a whole 256-wide chunk (block = L >> 2).
__device__ __forceinline__ void warp_pack_chunk(const float (&v)[8], uint8_t* rec)
{
    const int lane = threadIdx.x & 31;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const float inv = amax > 0.0f ? 32639.0f / amax : 0.0f;
    uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
    int bsum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int hi, lo;
        bsum += quant16(v[i], inv, hi, lo);
        hw[i >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (i & 3));
        lw[i >> 2] |= (uint32_t)(lo & 0xFF) << (8 * (i & 3));
    }
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 1);
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 2);
    // activations 8*part..8*part+7 of block b: fragment lanes t = 2*(part&1) and +1, word part>>1
    const int b = lane >> 2, part = lane & 3;
    uint32_t* xq = reinterpret_cast<uint32_t*>(rec + b * 64);
    const int t0 = 2 * (part & 1), half = part >> 1;
    xq[(0 * 4 + t0) * 2 + half] = hw[0];
    xq[(0 * 4 + t0 + 1) * 2 + half] = hw[1];
    xq[(1 * 4 + t0) * 2 + half] = lw[0];
    xq[(1 * 4 + t0 + 1) * 2 + half] = lw[1];
    if (part == 0) {
        reinterpret_cast<int4*>(rec + XPK1_META)[b] =
            make_int4(8 * bsum, 128 * bsum, __float_as_int(amax / 32639.0f), 0);
    }
}

}  // namespace
}  // namespace qmm

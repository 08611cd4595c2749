// Activation packing for the integer-MMA matvec and the dispatch of a matvec to the block
// format's kernels (qmm_gemv_kernel.cuh, instantiated per format in qmm_gemv_<format>.cu).
#include "qmm_gemv_device.cuh"
#include "qmm_kernels.h"
#include "qmm_pack.cuh"

namespace qmm {

namespace {

// Quantize x to 16 bits per (row, 32-wide block) and store it in B-fragment order
// (qmm_common.cuh).  grid (kc, ncp), 128 threads: warp w handles activation row 4*blockIdx.y + w
// of chunk blockIdx.x, lane L its columns 8L..8L+7 (block L >> 2).
__global__ void __launch_bounds__(128) pack_x_kernel(const float* __restrict__ x, int m, int64_t k, int ncp,
                                                     int compact, uint8_t* __restrict__ out)
{
    __shared__ short q[4][256];
    pdl_launch_dependents();  // the matvec that follows may start fetching its weights
    pdl_wait();               // x may come from the previous kernel; the buffer may still be read by it
    const int c = blockIdx.x;
    const int j = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int row = 4 * j + warp;

    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t col = (int64_t)c * 256 + 8 * lane + i;
        v[i] = (row < m && col < k) ? x[(int64_t)row * k + col] : 0.0f;
    }
    if (compact) {
        if (warp == 0) {
            warp_pack_chunk(v, out + (size_t)c * XPK1_REC);
        }
        return;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const float inv = amax > 0.0f ? 32639.0f / amax : 0.0f;
    int bsum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int hi, lo;
        const int qi = quant16(v[i], inv, hi, lo);
        q[warp][8 * lane + i] = (short)qi;
        bsum += qi;
    }
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 1);
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 2);
    uint8_t* rec = out + (size_t)c * xpack_rec_bytes(ncp);
    if ((lane & 3) == 0) {
        reinterpret_cast<int4*>(rec + xpack_xq_bytes(ncp))[(lane >> 2) * 16 + row] =
            make_int4(8 * bsum, 128 * bsum, __float_as_int(amax / 32639.0f), 0);
    }
    __syncthreads();

    // fragment lane (g,t) of block b: activation row g>>1 of this group, digit g&1 (0 = high byte)
    uint2* xq = reinterpret_cast<uint2*>(rec);
    for (int i = threadIdx.x; i < 8 * 32; i += 128) {
        const int b = i >> 5;
        const int fl = i & 31;
        const int g = fl >> 2;
        const int t = fl & 3;
        const int r = g >> 1;
        const int lo_digit = g & 1;
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int q0 = q[r][32 * b + 4 * t + e];
            const int q1 = q[r][32 * b + 16 + 4 * t + e];
            const int l0 = ((q0 + 128) & 0xFF) - 128;
            const int l1 = ((q1 + 128) & 0xFF) - 128;
            const int d0 = lo_digit ? l0 : ((q0 - l0) >> 8);
            const int d1 = lo_digit ? l1 : ((q1 - l1) >> 8);
            w0 |= (uint32_t)(d0 & 0xFF) << (8 * e);
            w1 |= (uint32_t)(d1 & 0xFF) << (8 * e);
        }
        xq[(size_t)(b * ncp + j) * 32 + fl] = make_uint2(w0, w1);
    }
}

// Inverse of the compact packing, for verification: x[i] = xs * (256*hi + lo).
__global__ void unpack_x_kernel(const uint8_t* __restrict__ packed, int64_t k, float* __restrict__ x)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < k; i += (int64_t)gridDim.x * blockDim.x) {
        const uint8_t* rec = packed + (size_t)(i >> 8) * XPK1_REC;
        const int b = (int)(i >> 5) & 7, e = (int)i & 31;
        const int half = e >> 4, t = (e & 15) >> 2, byte = e & 3;
        const uint32_t* xq = reinterpret_cast<const uint32_t*>(rec + b * 64);
        const int hi = (int)(signed char)((xq[(0 * 4 + t) * 2 + half] >> (8 * byte)) & 0xFFu);
        const int lo = (int)(signed char)((xq[(1 * 4 + t) * 2 + half] >> (8 * byte)) & 0xFFu);
        const float xs = __int_as_float(reinterpret_cast<const int4*>(rec + XPK1_META)[b].z);
        x[i] = xs * (float)(256 * hi + lo);
    }
}

// fp32 -> bf16 (round to nearest even), for fp32 callers of the prefill GEMM
__global__ void f32_to_bf16_kernel(const float* __restrict__ x, int64_t count, unsigned short* __restrict__ out)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t u = __float_as_uint(x[i]);
        const uint32_t r = (u & 0x7F800000u) == 0x7F800000u ? u : u + 0x7FFFu + ((u >> 16) & 1u);  // keeps inf/nan
        out[i] = (unsigned short)(r >> 16);
    }
}

}  // namespace

cudaError_t launch_f32_to_bf16(const float* x, int64_t count, void* out_bf16, cudaStream_t stream)
{
    const int64_t blocks = (count + 255) / 256;
    f32_to_bf16_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, stream>>>(x, count,
                                                                                      static_cast<unsigned short*>(out_bf16));
    return cudaGetLastError();
}

cudaError_t launch_pack_x(const float* x, int m, int64_t k, int kc, uint8_t* out, cudaStream_t stream)
{
    const int ncp = xpack_ncp(m);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)kc, (unsigned)ncp);
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, pack_x_kernel, x, m, k, ncp, m == 1 ? 1 : 0, out);
}

cudaError_t launch_unpack_x(const uint8_t* packed, int64_t k, float* x, cudaStream_t stream)
{
    unpack_x_kernel<<<(unsigned)((k + 255) / 256), 256, 0, stream>>>(packed, k, x);
    return cudaGetLastError();
}

cudaError_t launch_gemv_fused(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                              const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream)
{
    if ((ps.n_peers > 0 || fu.mode != EPI_STORE || fu.ss_in != nullptr || fu.x_f32 != nullptr) && m != 1) {
        return cudaErrorInvalidValue;
    }
    if (ps.n_peers > 0 && fu.mode != EPI_STORE &&
        !(fu.mode == EPI_RESID_PACK && ps.recv != nullptr && ps.wait_status != nullptr && ps.tp_size == ps.n_peers + 1)) {
        return cudaErrorInvalidValue;  // only the residual form also finishes the sum over the ranks
    }
    if ((fu.mode == EPI_RESID_PACK && w.n % 32 != 0) || (fu.mode == EPI_SWIGLU && w.n % 16 != 0) ||
        (fu.mode == EPI_SWIGLU_PACK && (w.n % 64 != 0 || fu.packed_out == nullptr)) || (fu.x_f32 && w.k % 32 != 0)) {
        return cudaErrorInvalidValue;
    }
    switch (w.fmt) {
    case FMT_Q4_0: return launch_gemv_q4_0(w, xp, y, m, status, ps, fu, stream);
    case FMT_Q8_0: return launch_gemv_q8_0(w, xp, y, m, status, ps, fu, stream);
    case FMT_Q4_K: return launch_gemv_q4_k(w, xp, y, m, status, ps, fu, stream);
    case FMT_Q6_K: return launch_gemv_q6_k(w, xp, y, m, status, ps, fu, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemv(const WeightView& w, const XPackView& xp, float* y, int m, int* status, cudaStream_t stream)
{
    const PeerScatter none = {};
    const GemvFuse plain = {};
    return launch_gemv_fused(w, xp, y, m, status, none, plain, stream);
}

}  // namespace qmm

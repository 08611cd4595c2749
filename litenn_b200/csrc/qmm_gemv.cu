// Dequant-fused GEMV / skinny GEMM for decode (1..16 activation rows) on sm_100a.
//
// The weights never become floats in memory.  Each warp streams 16-row x 256-column
// tiles of the packed weight (qmm_common.cuh) with 16-byte no-allocate loads — every
// request of a warp is one contiguous 512-byte segment — turns the quants into int8
// MMA A-fragments with two or three logic ops per word, and multiplies them on the
// integer tensor-core path (mma.sync m16n8k32 / m16n8k16, s32 accumulate) with the
// activations, which a small pre-pass has quantized to 16 bits per (row, 256 chunk)
// and split into a signed high and an unsigned low byte.  The int32 block sums are
// exact; they are folded into fp32 accumulators with the block's fp16 scale, so the
// accumulation across blocks is fp32 as in the reference loop
// (src/LiteNN/Device.h:645-658).  The only approximation is the 16-bit activation
// quantization (relative error <= 2^-16 of the chunk maximum).
//
// HBM-bound by design: per 32 weights a lane issues ~25-40 instructions, well under
// what the SM can issue in the time HBM needs to deliver those 18-34 bytes.
#include "qmm_kernels.h"

namespace qmm {

namespace {

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ uint16_t ldg_stream_u16(const void* p)
{
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// D = A(16x32, row) * B(32x8, col), s32 accumulators starting from zero.
template <bool A_SIGNED, bool B_SIGNED>
__device__ __forceinline__ void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1)
{
    c[0] = c[1] = c[2] = c[3] = 0;
    if constexpr (A_SIGNED && B_SIGNED) {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else if constexpr (A_SIGNED && !B_SIGNED) {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else if constexpr (!A_SIGNED && B_SIGNED) {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// D = A(16x16, row, s8) * B(16x8, col), s32 accumulators starting from zero.
template <bool B_SIGNED>
__device__ __forceinline__ void mma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    c[0] = c[1] = c[2] = c[3] = 0;
    if constexpr (B_SIGNED) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                     : "r"(a0), "r"(a1), "r"(b0));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                     : "r"(a0), "r"(a1), "r"(b0));
    }
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i)
{
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

__device__ __forceinline__ float half_of(const uint4& v, int b)
{
    const uint32_t w = word_of(v, b >> 1);
    return __half2float(__ushort_as_half((unsigned short)((b & 1) ? (w >> 16) : (w & 0xFFFFu))));
}

__device__ __forceinline__ uint32_t byte_of(const uint4& v, int i)
{
    return (word_of(v, i >> 2) >> (8 * (i & 3))) & 0xFFu;
}

// Registers one lane holds for one 16x256 tile.
template <int FMT>
struct ChunkData;
template <>
struct ChunkData<FMT_Q4_0> {
    uint4 q[4];
    uint4 s0, s1;
};
template <>
struct ChunkData<FMT_Q8_0> {
    uint4 q[8];
    uint4 s0, s1;
};
template <>
struct ChunkData<FMT_Q4_K> {
    uint4 q[4];
    uint4 s0, s1;
    uint32_t e0, e1;
};
template <>
struct ChunkData<FMT_Q6_K> {
    uint4 q[6];
    uint4 s0, s1;
    uint32_t e0, e1;
};

template <int FMT>
__device__ __forceinline__ void load_chunk(ChunkData<FMT>& cd, const WeightView& v, int64_t tile, int lane)
{
    constexpr int NQ = tile_qs_bytes(FMT) / 512;
    const int g = lane >> 2;
    const uint8_t* qs = v.qs + tile * tile_qs_bytes(FMT) + lane * 16;
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
        cd.q[i] = ldg_stream_v4(qs + i * 512);
    }
    const uint8_t* p1 = v.p1 + tile * 256;
    cd.s0 = ldg_stream_v4(p1 + g * 16);
    cd.s1 = ldg_stream_v4(p1 + (g + 8) * 16);
    if constexpr (FMT == FMT_Q4_K) {
        cd.e0 = ldg_stream_u32(v.p2 + tile * 64 + g * 4);
        cd.e1 = ldg_stream_u32(v.p2 + tile * 64 + (g + 8) * 4);
    }
    if constexpr (FMT == FMT_Q6_K) {
        cd.e0 = ldg_stream_u16(v.p2 + tile * 32 + g * 2);
        cd.e1 = ldg_stream_u16(v.p2 + tile * 32 + (g + 8) * 2);
    }
}

// MC = activation columns handled: 1 (only column 0 is live), 8 or 16.
template <int MC>
struct Cols {
    static constexpr int NCG = MC == 16 ? 2 : 1;
    static constexpr int NOUT = MC == 1 ? 2 : 4 * NCG;
};

template <int MC>
__device__ __forceinline__ uint4 load_xfrag(const XPackView& xp, int c, int b, int cgi, int lane)
{
    const uint4* p = xp.xq + ((size_t)(c * 8 + b) * xp.cg + cgi) * 32 + lane;
    if constexpr (MC == 1) {
        // only activation row 0 is live: lanes 0..3 (g == 0) carry it
        uint4 z = make_uint4(0u, 0u, 0u, 0u);
        if (lane < 4) {
            z = __ldg(p);
        }
        return z;
    } else {
        return __ldg(p);
    }
}

// accc += (256*hi + lo) * row scale
template <int MC>
__device__ __forceinline__ void fold(float* accc, int cgi, const int (&chi)[4], const int (&clo)[4], float sg,
                                     float sg8)
{
    if constexpr (MC == 1) {
        accc[0] = fmaf((float)(chi[0] * 256 + clo[0]), sg, accc[0]);
        accc[1] = fmaf((float)(chi[2] * 256 + clo[2]), sg8, accc[1]);
    } else {
        float* a = accc + 4 * cgi;
        a[0] = fmaf((float)(chi[0] * 256 + clo[0]), sg, a[0]);
        a[1] = fmaf((float)(chi[1] * 256 + clo[1]), sg, a[1]);
        a[2] = fmaf((float)(chi[2] * 256 + clo[2]), sg8, a[2]);
        a[3] = fmaf((float)(chi[3] * 256 + clo[3]), sg8, a[3]);
    }
}

// acc += accc * (activation scale of the chunk) * extra
template <int MC>
__device__ __forceinline__ void fold_chunk(float* acc, const float* accc, const XPackView& xp, int c, int lane,
                                           float extra)
{
    const int t = lane & 3;
    if constexpr (MC == 1) {
        const float sx = __ldg(xp.xs + c * 16) * extra;
        acc[0] = fmaf(accc[0], sx, acc[0]);
        acc[1] = fmaf(accc[1], sx, acc[1]);
    } else {
#pragma unroll
        for (int cgi = 0; cgi < Cols<MC>::NCG; ++cgi) {
            const float2 sx = __ldg(reinterpret_cast<const float2*>(xp.xs + c * 16 + 8 * cgi + 2 * t));
            const float s0 = sx.x * extra;
            const float s1 = sx.y * extra;
            acc[4 * cgi + 0] = fmaf(accc[4 * cgi + 0], s0, acc[4 * cgi + 0]);
            acc[4 * cgi + 1] = fmaf(accc[4 * cgi + 1], s1, acc[4 * cgi + 1]);
            acc[4 * cgi + 2] = fmaf(accc[4 * cgi + 2], s0, acc[4 * cgi + 2]);
            acc[4 * cgi + 3] = fmaf(accc[4 * cgi + 3], s1, acc[4 * cgi + 3]);
        }
    }
}

template <int FMT, int MC>
__device__ __forceinline__ void compute_chunk(const ChunkData<FMT>& cd, const XPackView& xp, int c, int lane,
                                              float* acc)
{
    constexpr int NCG = Cols<MC>::NCG;
    constexpr int NOUT = Cols<MC>::NOUT;
    float accc[NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
        accc[o] = 0.0f;
    }
    int chi[4], clo[4];

    if constexpr (FMT == FMT_Q4_0) {
        // A byte = (nibble << 4) ^ 0x80 = 16 * (nibble - 8) as int8: no offset term left.
#pragma unroll
        for (int p = 0; p < 4; ++p) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t wa = h ? cd.q[p].z : cd.q[p].x;
                const uint32_t wb = h ? cd.q[p].w : cd.q[p].y;
                const uint32_t a0 = ((wa << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                const uint32_t a2 = (wa & 0xF0F0F0F0u) ^ 0x80808080u;
                const uint32_t a1 = ((wb << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                const uint32_t a3 = (wb & 0xF0F0F0F0u) ^ 0x80808080u;
                const int b = 2 * p + h;
                const float dg = half_of(cd.s0, b);
                const float dg8 = half_of(cd.s1, b);
#pragma unroll
                for (int cgi = 0; cgi < NCG; ++cgi) {
                    const uint4 xf = load_xfrag<MC>(xp, c, b, cgi, lane);
                    mma_k32<true, true>(chi, a0, a1, a2, a3, xf.x, xf.y);
                    mma_k32<true, false>(clo, a0, a1, a2, a3, xf.z, xf.w);
                    fold<MC>(accc, cgi, chi, clo, dg, dg8);
                }
            }
        }
        fold_chunk<MC>(acc, accc, xp, c, lane, 0.0625f);
    } else if constexpr (FMT == FMT_Q8_0) {
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const float dg = half_of(cd.s0, b);
            const float dg8 = half_of(cd.s1, b);
#pragma unroll
            for (int cgi = 0; cgi < NCG; ++cgi) {
                const uint4 xf = load_xfrag<MC>(xp, c, b, cgi, lane);
                mma_k32<true, true>(chi, cd.q[b].x, cd.q[b].y, cd.q[b].z, cd.q[b].w, xf.x, xf.y);
                mma_k32<true, false>(clo, cd.q[b].x, cd.q[b].y, cd.q[b].z, cd.q[b].w, xf.z, xf.w);
                fold<MC>(accc, cgi, chi, clo, dg, dg8);
            }
        }
        fold_chunk<MC>(acc, accc, xp, c, lane, 1.0f);
    } else if constexpr (FMT == FMT_Q4_K) {
        const int t = lane & 3;
        const float dg = __half2float(__ushort_as_half((unsigned short)(cd.e0 & 0xFFFFu)));
        const float ming = __half2float(__ushort_as_half((unsigned short)(cd.e0 >> 16)));
        const float dg8 = __half2float(__ushort_as_half((unsigned short)(cd.e1 & 0xFFFFu)));
        const float ming8 = __half2float(__ushort_as_half((unsigned short)(cd.e1 >> 16)));
#pragma unroll
        for (int p = 0; p < 4; ++p) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int sb = 2 * p + h;
                const int sh = 4 * h;
                const uint32_t a0 = (cd.q[p].x >> sh) & 0x0F0F0F0Fu;
                const uint32_t a1 = (cd.q[p].y >> sh) & 0x0F0F0F0Fu;
                const uint32_t a2 = (cd.q[p].z >> sh) & 0x0F0F0F0Fu;
                const uint32_t a3 = (cd.q[p].w >> sh) & 0x0F0F0F0Fu;
                const float sg = dg * (float)byte_of(cd.s0, sb);
                const float sg8 = dg8 * (float)byte_of(cd.s1, sb);
                const float mg = ming * (float)byte_of(cd.s0, 8 + sb);
                const float mg8 = ming8 * (float)byte_of(cd.s1, 8 + sb);
#pragma unroll
                for (int cgi = 0; cgi < NCG; ++cgi) {
                    const uint4 xf = load_xfrag<MC>(xp, c, sb, cgi, lane);
                    mma_k32<false, true>(chi, a0, a1, a2, a3, xf.x, xf.y);
                    mma_k32<false, false>(clo, a0, a1, a2, a3, xf.z, xf.w);
                    fold<MC>(accc, cgi, chi, clo, sg, sg8);
                    // the "- dmin*m" part of every weight times the plain sum of the block's activations
                    const float* xsum = xp.xsum + (size_t)(c * 8 + sb) * 16;
                    if constexpr (MC == 1) {
                        const float s = __ldg(xsum);
                        acc[0] = fmaf(-mg, s, acc[0]);
                        acc[1] = fmaf(-mg8, s, acc[1]);
                    } else {
                        const float2 s = __ldg(reinterpret_cast<const float2*>(xsum + 8 * cgi + 2 * t));
                        acc[4 * cgi + 0] = fmaf(-mg, s.x, acc[4 * cgi + 0]);
                        acc[4 * cgi + 1] = fmaf(-mg, s.y, acc[4 * cgi + 1]);
                        acc[4 * cgi + 2] = fmaf(-mg8, s.x, acc[4 * cgi + 2]);
                        acc[4 * cgi + 3] = fmaf(-mg8, s.y, acc[4 * cgi + 3]);
                    }
                }
            }
        }
        fold_chunk<MC>(acc, accc, xp, c, lane, 1.0f);
    } else {  // Q6_K: A byte = 4 * (q - 32) as int8, one k16 MMA per 16-wide sub-block
        const float dg = __half2float(__ushort_as_half((unsigned short)cd.e0));
        const float dg8 = __half2float(__ushort_as_half((unsigned short)cd.e1));
#pragma unroll
        for (int quad = 0; quad < 4; ++quad) {
            uint32_t out[2][4];
#pragma unroll
            for (int rsel = 0; rsel < 2; ++rsel) {
                const int base = (quad * 2 + rsel) * 3;
                const uint32_t X = word_of(cd.q[(base + 0) >> 2], (base + 0) & 3);
                const uint32_t Y = word_of(cd.q[(base + 1) >> 2], (base + 1) & 3);
                const uint32_t Z = word_of(cd.q[(base + 2) >> 2], (base + 2) & 3);
                out[rsel][0] = X & 0xFCFCFCFCu;
                out[rsel][1] = Y & 0xFCFCFCFCu;
                out[rsel][2] = Z & 0xFCFCFCFCu;
                out[rsel][3] = ((X & 0x03030303u) << 6) | ((Y & 0x03030303u) << 4) | ((Z & 0x03030303u) << 2);
            }
#pragma unroll
            for (int cgi = 0; cgi < NCG; ++cgi) {
                const uint4 xf0 = load_xfrag<MC>(xp, c, 2 * quad, cgi, lane);
                const uint4 xf1 = load_xfrag<MC>(xp, c, 2 * quad + 1, cgi, lane);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int sb = 4 * quad + j;
                    const uint4& xf = (j >> 1) ? xf1 : xf0;
                    const uint32_t bhi = (j & 1) ? xf.y : xf.x;
                    const uint32_t blo = (j & 1) ? xf.w : xf.z;
                    mma_k16<true>(chi, out[0][j], out[1][j], bhi);
                    mma_k16<false>(clo, out[0][j], out[1][j], blo);
                    const float sg = dg * (float)(int)(signed char)byte_of(cd.s0, sb);
                    const float sg8 = dg8 * (float)(int)(signed char)byte_of(cd.s1, sb);
                    fold<MC>(accc, cgi, chi, clo, sg, sg8);
                }
            }
        }
        fold_chunk<MC>(acc, accc, xp, c, lane, 0.25f);
    }
}

// One CTA per 16-row tile; its WARPS warps take the K chunks round-robin and the
// partial sums meet in shared memory.
template <int FMT, int MC, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) gemv_kernel(WeightView v, XPackView xp, float* __restrict__ y, int m)
{
    constexpr int NOUT = Cols<MC>::NOUT;
    __shared__ float red[WARPS][16][MC];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t tile0 = (int64_t)blockIdx.x * v.kc;

    float acc[NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
        acc[o] = 0.0f;
    }

    ChunkData<FMT> cur, nxt;
    int c = warp;
    if (c < v.kc) {
        load_chunk<FMT>(cur, v, tile0 + c, lane);
    }
    for (; c < v.kc; c += WARPS) {
        const int cn = c + WARPS;
        if (cn < v.kc) {
            load_chunk<FMT>(nxt, v, tile0 + cn, lane);
        }
        compute_chunk<FMT, MC>(cur, xp, c, lane, acc);
        cur = nxt;
    }

    const int g = lane >> 2;
    const int t = lane & 3;
    if constexpr (MC == 1) {
        if (t == 0) {
            red[warp][g][0] = acc[0];
            red[warp][g + 8][0] = acc[1];
        }
    } else {
#pragma unroll
        for (int cgi = 0; cgi < Cols<MC>::NCG; ++cgi) {
            red[warp][g][8 * cgi + 2 * t] = acc[4 * cgi + 0];
            red[warp][g][8 * cgi + 2 * t + 1] = acc[4 * cgi + 1];
            red[warp][g + 8][8 * cgi + 2 * t] = acc[4 * cgi + 2];
            red[warp][g + 8][8 * cgi + 2 * t + 1] = acc[4 * cgi + 3];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * MC; i += WARPS * 32) {
        const int col = i >> 4;
        const int r = i & 15;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            s += red[w][r][col];
        }
        const int64_t row = (int64_t)blockIdx.x * 16 + r;
        if (row < v.n && col < m) {
            y[(int64_t)col * v.n + row] = s;
        }
    }
}

// Quantize x to 16 bits per (row, 256-chunk) and store it in B-fragment order.
// grid (kc, cg), 256 threads: warp w handles activation row 8*cg_index + w.
__global__ void __launch_bounds__(256) pack_x_kernel(const float* __restrict__ x, int m, int64_t k, int cg,
                                                     uint4* __restrict__ xq, float* __restrict__ xs,
                                                     float* __restrict__ xsum)
{
    __shared__ short q[8][256];
    const int c = blockIdx.x;
    const int cgi = blockIdx.y;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int row = 8 * cgi + warp;

    float v[8];
    float amax = 0.0f;
    float bsum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t col = (int64_t)c * 256 + 8 * lane + i;
        v[i] = (row < m && col < k) ? x[(int64_t)row * k + col] : 0.0f;
        amax = fmaxf(amax, fabsf(v[i]));
        bsum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    }
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 1);
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 2);
    const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int qi = __float2int_rn(v[i] * inv);
        qi = max(-32767, min(32767, qi));
        q[warp][8 * lane + i] = (short)qi;
    }
    if (lane == 0) {
        xs[c * 16 + row] = amax / 32767.0f;
    }
    if ((lane & 3) == 0) {
        xsum[(size_t)(c * 8 + (lane >> 2)) * 16 + row] = bsum;
    }
    __syncthreads();

    // thread -> (block b, fragment lane L)
    const int b = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    uint32_t hi0 = 0, hi1 = 0, lo0 = 0, lo1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q0 = q[g][32 * b + 4 * t + i];
        const int q1 = q[g][32 * b + 16 + 4 * t + i];
        hi0 |= (uint32_t)((q0 >> 8) & 0xFF) << (8 * i);
        lo0 |= (uint32_t)(q0 & 0xFF) << (8 * i);
        hi1 |= (uint32_t)((q1 >> 8) & 0xFF) << (8 * i);
        lo1 |= (uint32_t)(q1 & 0xFF) << (8 * i);
    }
    xq[((size_t)(c * 8 + b) * cg + cgi) * 32 + lane] = make_uint4(hi0, hi1, lo0, lo1);
}

template <int FMT, int MC>
cudaError_t launch_gemv_fmt_mc(const WeightView& w, const XPackView& xp, float* y, int m, cudaStream_t stream)
{
    if (w.kc >= 32) {
        gemv_kernel<FMT, MC, 8><<<w.rt, 256, 0, stream>>>(w, xp, y, m);
    } else {
        gemv_kernel<FMT, MC, 4><<<w.rt, 128, 0, stream>>>(w, xp, y, m);
    }
    return cudaGetLastError();
}

template <int FMT>
cudaError_t launch_gemv_fmt(const WeightView& w, const XPackView& xp, float* y, int m, cudaStream_t stream)
{
    if (m == 1) {
        return launch_gemv_fmt_mc<FMT, 1>(w, xp, y, m, stream);
    }
    if (m <= 8) {
        return launch_gemv_fmt_mc<FMT, 8>(w, xp, y, m, stream);
    }
    return launch_gemv_fmt_mc<FMT, 16>(w, xp, y, m, stream);
}

}  // namespace

cudaError_t launch_pack_x(const float* x, int m, int64_t k, int kc, int cg, const XPackBuffers& out,
                          cudaStream_t stream)
{
    pack_x_kernel<<<dim3(kc, cg), 256, 0, stream>>>(x, m, k, cg, out.xq, out.xs, out.xsum);
    return cudaGetLastError();
}

cudaError_t launch_gemv(const WeightView& w, const XPackView& xp, float* y, int m, int sm_count,
                        cudaStream_t stream)
{
    (void)sm_count;
    switch (w.fmt) {
    case FMT_Q4_0: return launch_gemv_fmt<FMT_Q4_0>(w, xp, y, m, stream);
    case FMT_Q8_0: return launch_gemv_fmt<FMT_Q8_0>(w, xp, y, m, stream);
    case FMT_Q4_K: return launch_gemv_fmt<FMT_Q4_K>(w, xp, y, m, stream);
    case FMT_Q6_K: return launch_gemv_fmt<FMT_Q6_K>(w, xp, y, m, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace qmm

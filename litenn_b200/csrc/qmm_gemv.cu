// Dequant-fused GEMV / skinny GEMM for decode (1..16 activation rows) on sm_100a.
//
// The weights never become floats in memory.  One CTA owns one 16-row tile of the
// output; its warps take the 256-column K chunks of that row tile round-robin.
// Every chunk is one contiguous packed tile (qmm_common.cuh) that a single TMA bulk
// copy (cp.async.bulk, completion counted on an mbarrier) lands in a shared-memory
// slot.  Each warp owns DEPTH slots and refills a slot itself as soon as it has
// consumed it, so the copies of a whole CTA (~36 KB) are in flight from the first
// instruction on and HBM latency is paid once, not per chunk.  From shared memory
// the quants become int8 MMA A-fragments with two or three logic ops per word and
// are multiplied on the integer tensor-core path (mma.sync m16n8k32 / m16n8k16, s32
// accumulate) with the activations, quantized to 16 bits per (row, 256 chunk) and
// split into a signed high and an unsigned low byte.  The int32 block sums are
// exact; they are folded into fp32 accumulators with the block's fp16 scale, so the
// accumulation across blocks is fp32 as in the reference loop
// (src/LiteNN/Device.h:645-658).  The only approximation is the 16-bit activation
// quantization (relative error <= 2^-16 of the chunk maximum).
//
// Batch 1 quantizes the activation vector inside the kernel (each warp the chunks
// it will consume, while its first weight tiles are in flight); batches 2..16 read
// activations packed by pack_x_kernel.  Kernels are launched with programmatic
// dependent launch: the weight copies are issued before griddepcontrol.wait, so in
// a chain of dependent matvecs the next kernel's weights stream while the previous
// kernel drains.
#include "qmm_kernels.h"

namespace qmm {

namespace {

// ---- PTX helpers ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// Global -> shared bulk copy; `bytes` and both addresses are multiples of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Bounded wait for a phase of an mbarrier.  Returns false when the limit ran out
// (the caller records an error status and stops using the pipeline).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) {
            return true;
        }
    }
    return false;
}

__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
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

__device__ __forceinline__ uint32_t byte_of_word(uint32_t w, int i)
{
    return (w >> (8 * i)) & 0xFFu;
}

// ---- activation sources -------------------------------------------------------------------

// MC = activation columns handled: 1 (only column 0 is live), 8 or 16.
template <int MC>
struct Cols {
    static constexpr int NCG = MC == 16 ? 2 : 1;
    static constexpr int NOUT = MC == 1 ? 2 : 4 * NCG;
};

// Batch 1: activations quantized by this CTA into shared memory.
//   xq   [kc][8 blocks][4 t] uint4 {hi k 4t.., hi k 16+4t.., lo k 4t.., lo k 16+4t..}
//   xs   [kc]  scale of the chunk;  xsum [kc][8] plain sum of each 32-block
struct XShared {
    const uint4* xq;
    const float* xs;
    const float* xsum;
    __device__ __forceinline__ uint4 frag(int c, int b, int /*cgi*/, int lane) const
    {
        // only activation row 0 is live: lanes 0..3 (g == 0) carry it
        return lane < 4 ? xq[(c * 8 + b) * 4 + lane] : make_uint4(0u, 0u, 0u, 0u);
    }
};

// Batches 2..16: activations packed in global memory by pack_x_kernel.
struct XGlobal {
    XPackView xp;
    __device__ __forceinline__ uint4 frag(int c, int b, int cgi, int lane) const
    {
        return __ldg(xp.xq + ((size_t)(c * 8 + b) * xp.cg + cgi) * 32 + lane);
    }
};

template <int MC>
using XSrc = typename std::conditional<MC == 1, XShared, XGlobal>::type;

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
__device__ __forceinline__ void fold_chunk(float* acc, const float* accc, const XSrc<MC>& xs, int c, int lane,
                                           float extra)
{
    if constexpr (MC == 1) {
        const float sx = xs.xs[c] * extra;
        acc[0] = fmaf(accc[0], sx, acc[0]);
        acc[1] = fmaf(accc[1], sx, acc[1]);
    } else {
        const int t = lane & 3;
#pragma unroll
        for (int cgi = 0; cgi < Cols<MC>::NCG; ++cgi) {
            const float2 sx = __ldg(reinterpret_cast<const float2*>(xs.xp.xs + c * 16 + 8 * cgi + 2 * t));
            const float s0 = sx.x * extra;
            const float s1 = sx.y * extra;
            acc[4 * cgi + 0] = fmaf(accc[4 * cgi + 0], s0, acc[4 * cgi + 0]);
            acc[4 * cgi + 1] = fmaf(accc[4 * cgi + 1], s1, acc[4 * cgi + 1]);
            acc[4 * cgi + 2] = fmaf(accc[4 * cgi + 2], s0, acc[4 * cgi + 2]);
            acc[4 * cgi + 3] = fmaf(accc[4 * cgi + 3], s1, acc[4 * cgi + 3]);
        }
    }
}

// The "- dmin*m" part of Q4_K: every weight of the block carries the same offset,
// so it multiplies the plain sum of the block's activations.
template <int MC>
__device__ __forceinline__ void fold_min(float* acc, const XSrc<MC>& xs, int c, int sb, int cgi, int lane, float mg,
                                         float mg8)
{
    if constexpr (MC == 1) {
        const float s = xs.xsum[c * 8 + sb];
        acc[0] = fmaf(-mg, s, acc[0]);
        acc[1] = fmaf(-mg8, s, acc[1]);
    } else {
        const int t = lane & 3;
        const float2 s =
            __ldg(reinterpret_cast<const float2*>(xs.xp.xsum + (size_t)(c * 8 + sb) * 16 + 8 * cgi + 2 * t));
        acc[4 * cgi + 0] = fmaf(-mg, s.x, acc[4 * cgi + 0]);
        acc[4 * cgi + 1] = fmaf(-mg, s.y, acc[4 * cgi + 1]);
        acc[4 * cgi + 2] = fmaf(-mg8, s.x, acc[4 * cgi + 2]);
        acc[4 * cgi + 3] = fmaf(-mg8, s.y, acc[4 * cgi + 3]);
    }
}

// One 16x256 tile, resident in shared memory at `slot`, times the activations of chunk c.
template <int FMT, int MC>
__device__ __forceinline__ void compute_chunk(const uint8_t* slot, const XSrc<MC>& xs, int c, int lane, float* acc)
{
    constexpr int NCG = Cols<MC>::NCG;
    constexpr int NOUT = Cols<MC>::NOUT;
    const int g = lane >> 2;
    float accc[NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
        accc[o] = 0.0f;
    }
    int chi[4], clo[4];
    const uint4* qs = reinterpret_cast<const uint4*>(slot) + lane;
    const uint8_t* p1 = slot + tile_p1_offset(FMT);
    const uint8_t* p2 = slot + tile_p2_offset(FMT);

    if constexpr (FMT == FMT_Q4_0) {
        // A byte = (nibble << 4) ^ 0x80 = 16 * (nibble - 8) as int8: no offset term left.
        const uint4 s0 = *reinterpret_cast<const uint4*>(p1 + g * 16);
        const uint4 s1 = *reinterpret_cast<const uint4*>(p1 + (g + 8) * 16);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint4 q = qs[p * 32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t wa = h ? q.z : q.x;
                const uint32_t wb = h ? q.w : q.y;
                const uint32_t a0 = ((wa << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                const uint32_t a2 = (wa & 0xF0F0F0F0u) ^ 0x80808080u;
                const uint32_t a1 = ((wb << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
                const uint32_t a3 = (wb & 0xF0F0F0F0u) ^ 0x80808080u;
                const int b = 2 * p + h;
                const float dg = half_of(s0, b);
                const float dg8 = half_of(s1, b);
#pragma unroll
                for (int cgi = 0; cgi < NCG; ++cgi) {
                    const uint4 xf = xs.frag(c, b, cgi, lane);
                    mma_k32<true, true>(chi, a0, a1, a2, a3, xf.x, xf.y);
                    mma_k32<true, false>(clo, a0, a1, a2, a3, xf.z, xf.w);
                    fold<MC>(accc, cgi, chi, clo, dg, dg8);
                }
            }
        }
        fold_chunk<MC>(acc, accc, xs, c, lane, 0.0625f);
    } else if constexpr (FMT == FMT_Q8_0) {
        const uint4 s0 = *reinterpret_cast<const uint4*>(p1 + g * 16);
        const uint4 s1 = *reinterpret_cast<const uint4*>(p1 + (g + 8) * 16);
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const uint4 q = qs[b * 32];
            const float dg = half_of(s0, b);
            const float dg8 = half_of(s1, b);
#pragma unroll
            for (int cgi = 0; cgi < NCG; ++cgi) {
                const uint4 xf = xs.frag(c, b, cgi, lane);
                mma_k32<true, true>(chi, q.x, q.y, q.z, q.w, xf.x, xf.y);
                mma_k32<true, false>(clo, q.x, q.y, q.z, q.w, xf.z, xf.w);
                fold<MC>(accc, cgi, chi, clo, dg, dg8);
            }
        }
        fold_chunk<MC>(acc, accc, xs, c, lane, 1.0f);
    } else if constexpr (FMT == FMT_Q4_K) {
        // 12 packed bytes per row -> eight 6-bit scales and eight 6-bit mins, four per word
        uint32_t scw[2][2], mnw[2][2];
        float dd[2], dmin[2];
#pragma unroll
        for (int rs = 0; rs < 2; ++rs) {
            const uint32_t* sp = reinterpret_cast<const uint32_t*>(p1 + (g + 8 * rs) * 12);
            const uint32_t w0 = sp[0], w1 = sp[1], w2 = sp[2];
            scw[rs][0] = w0 & 0x3F3F3F3Fu;
            mnw[rs][0] = w1 & 0x3F3F3F3Fu;
            scw[rs][1] = (w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u);
            mnw[rs][1] = ((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u);
            const uint32_t dm = *reinterpret_cast<const uint32_t*>(p2 + (g + 8 * rs) * 4);
            dd[rs] = __half2float(__ushort_as_half((unsigned short)(dm & 0xFFFFu)));
            dmin[rs] = __half2float(__ushort_as_half((unsigned short)(dm >> 16)));
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint4 q = qs[p * 32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int sb = 2 * p + h;
                const int sh = 4 * h;
                const uint32_t a0 = (q.x >> sh) & 0x0F0F0F0Fu;
                const uint32_t a1 = (q.y >> sh) & 0x0F0F0F0Fu;
                const uint32_t a2 = (q.z >> sh) & 0x0F0F0F0Fu;
                const uint32_t a3 = (q.w >> sh) & 0x0F0F0F0Fu;
                const float sg = dd[0] * (float)byte_of_word(scw[0][sb >> 2], sb & 3);
                const float sg8 = dd[1] * (float)byte_of_word(scw[1][sb >> 2], sb & 3);
                const float mg = dmin[0] * (float)byte_of_word(mnw[0][sb >> 2], sb & 3);
                const float mg8 = dmin[1] * (float)byte_of_word(mnw[1][sb >> 2], sb & 3);
#pragma unroll
                for (int cgi = 0; cgi < NCG; ++cgi) {
                    const uint4 xf = xs.frag(c, sb, cgi, lane);
                    mma_k32<false, true>(chi, a0, a1, a2, a3, xf.x, xf.y);
                    mma_k32<false, false>(clo, a0, a1, a2, a3, xf.z, xf.w);
                    fold<MC>(accc, cgi, chi, clo, sg, sg8);
                    fold_min<MC>(acc, xs, c, sb, cgi, lane, mg, mg8);
                }
            }
        }
        fold_chunk<MC>(acc, accc, xs, c, lane, 1.0f);
    } else {  // Q6_K: A byte = 4 * (q - 32) as int8, one k16 MMA per 16-wide sub-block
        const uint4 s0 = *reinterpret_cast<const uint4*>(p1 + g * 16);
        const uint4 s1 = *reinterpret_cast<const uint4*>(p1 + (g + 8) * 16);
        const float dg = __half2float(*reinterpret_cast<const __half*>(p2 + g * 2));
        const float dg8 = __half2float(*reinterpret_cast<const __half*>(p2 + (g + 8) * 2));
        uint4 qv[6];
#pragma unroll
        for (int i = 0; i < 6; ++i) {
            qv[i] = qs[i * 32];
        }
#pragma unroll
        for (int quad = 0; quad < 4; ++quad) {
            uint32_t out[2][4];
#pragma unroll
            for (int rsel = 0; rsel < 2; ++rsel) {
                const int base = (quad * 2 + rsel) * 3;
                const uint32_t X = word_of(qv[(base + 0) >> 2], (base + 0) & 3);
                const uint32_t Y = word_of(qv[(base + 1) >> 2], (base + 1) & 3);
                const uint32_t Z = word_of(qv[(base + 2) >> 2], (base + 2) & 3);
                out[rsel][0] = X & 0xFCFCFCFCu;
                out[rsel][1] = Y & 0xFCFCFCFCu;
                out[rsel][2] = Z & 0xFCFCFCFCu;
                out[rsel][3] = ((X & 0x03030303u) << 6) | ((Y & 0x03030303u) << 4) | ((Z & 0x03030303u) << 2);
            }
#pragma unroll
            for (int cgi = 0; cgi < NCG; ++cgi) {
                const uint4 xf0 = xs.frag(c, 2 * quad, cgi, lane);
                const uint4 xf1 = xs.frag(c, 2 * quad + 1, cgi, lane);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int sb = 4 * quad + j;
                    const uint4& xf = (j >> 1) ? xf1 : xf0;
                    const uint32_t bhi = (j & 1) ? xf.y : xf.x;
                    const uint32_t blo = (j & 1) ? xf.w : xf.z;
                    mma_k16<true>(chi, out[0][j], out[1][j], bhi);
                    mma_k16<false>(clo, out[0][j], out[1][j], blo);
                    const float sg = dg * (float)(int)(signed char)byte_of(s0, sb);
                    const float sg8 = dg8 * (float)(int)(signed char)byte_of(s1, sb);
                    fold<MC>(accc, cgi, chi, clo, sg, sg8);
                }
            }
        }
        fold_chunk<MC>(acc, accc, xs, c, lane, 0.25f);
    }
}

// ---- in-kernel activation quantization (batch 1) ------------------------------------------

// Quantizes chunk c of the activation row x (k values) into the shared arrays.  Lane L
// holds elements 8L..8L+7 of the chunk: block L>>2, k-slots 8*(L&3)..+7 of that block.
__device__ __forceinline__ void quantize_chunk_to_smem(const float (&v)[8], int c, int lane, uint32_t* xq_words,
                                                       float* xs, float* xsum)
{
    float amax = 0.0f;
    float bsum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
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
    uint32_t hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int qi = __float2int_rn(v[i] * inv);
        qi = max(-32767, min(32767, qi));
        hi[i >> 2] |= (uint32_t)((qi >> 8) & 0xFF) << (8 * (i & 3));
        lo[i >> 2] |= (uint32_t)(qi & 0xFF) << (8 * (i & 3));
    }
    // k-slots 8*(L&3)+{0..3} -> fragment lane t = 2*((L&3)&1), +{4..7} -> t+1;
    // (L&3)>>1 selects the b0 (slots 0..15) or b1 (slots 16..31) register.
    const int b = lane >> 2;
    const int part = lane & 3;
    const int half = part >> 1;
    const int t0 = 2 * (part & 1);
    uint32_t* base = xq_words + ((size_t)(c * 8 + b) * 4) * 4;
    base[(t0 + 0) * 4 + half] = hi[0];
    base[(t0 + 0) * 4 + 2 + half] = lo[0];
    base[(t0 + 1) * 4 + half] = hi[1];
    base[(t0 + 1) * 4 + 2 + half] = lo[1];
    if (lane == 0) {
        xs[c] = amax / 32767.0f;
    }
    if (part == 0) {
        xsum[c * 8 + b] = bsum;
    }
}

__device__ __forceinline__ void load_x_chunk(float (&v)[8], const float* __restrict__ x, int64_t k, int c, int lane,
                                             bool aligned)
{
    const int64_t col = (int64_t)c * 256 + 8 * lane;
    if (col + 8 <= k) {  // k is a multiple of 32, so a lane's 8 values are all in or all out
        if (aligned) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(x + col));
            const float4 b = __ldg(reinterpret_cast<const float4*>(x + col + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = __ldg(x + col + i);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = 0.0f;
        }
    }
}

// ---- the kernel -----------------------------------------------------------------------------

// Shared memory of one CTA, carved from the dynamic allocation:
//   slots  WARPS*DEPTH tiles | mbarriers | (batch 1) xq, xs, xsum | cross-warp reduction
template <int FMT, int WARPS, int DEPTH>
struct SmemPlan {
    static constexpr int SLOT = tile_bytes(FMT);
    static constexpr int SLOTS_BYTES = WARPS * DEPTH * SLOT;
    static constexpr int BAR_OFF = SLOTS_BYTES;
    static constexpr int BAR_BYTES = ((WARPS * DEPTH * 8 + 15) / 16) * 16;
    static constexpr int X_OFF = BAR_OFF + BAR_BYTES;
    __host__ __device__ static int xq_bytes(int kc) { return kc * 8 * 64; }
    __host__ __device__ static int xs_bytes(int kc) { return ((kc * 4 + 15) / 16) * 16; }
    __host__ __device__ static int xsum_bytes(int kc) { return kc * 8 * 4; }
    __host__ __device__ static int total(int kc, int mc)
    {
        const int x = mc == 1 ? xq_bytes(kc) + xs_bytes(kc) + xsum_bytes(kc) : 0;
        return X_OFF + x + WARPS * 16 * mc * 4;
    }
};

template <int FMT, int MC, int WARPS, int DEPTH>
__global__ void __launch_bounds__(WARPS * 32)
    gemv_kernel(WeightView v, const float* __restrict__ x, XPackView xp, float* __restrict__ y, int m,
                int* __restrict__ status)
{
    using Plan = SmemPlan<FMT, WARPS, DEPTH>;
    constexpr int NOUT = Cols<MC>::NOUT;
    constexpr uint32_t TILE = tile_bytes(FMT);
    extern __shared__ __align__(128) uint8_t smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int kc = v.kc;
    uint8_t* my_slots = smem + (size_t)warp * DEPTH * Plan::SLOT;
    uint64_t* my_bars = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFF) + warp * DEPTH;
    const uint8_t* my_tiles = v.tiles + (size_t)blockIdx.x * kc * TILE;
    const int n_my = warp < kc ? (kc - warp + WARPS - 1) / WARPS : 0;

    // 1. start the weight stream: the first DEPTH tiles of this warp
    if (lane == 0) {
        for (int s = 0; s < DEPTH; ++s) {
            mbar_init(&my_bars[s], 1);
        }
        fence_barrier_init();
        for (int s = 0; s < DEPTH && s < n_my; ++s) {
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)(warp + s * WARPS) * TILE, TILE,
                          &my_bars[s]);
        }
    }
    pdl_launch_dependents();
    // 2. everything below may read what the previous kernel in the stream produced
    pdl_wait();
    __syncwarp();

    XSrc<MC> xsrc;
    if constexpr (MC == 1) {
        uint8_t* xbase = smem + Plan::X_OFF;
        uint32_t* xq_words = reinterpret_cast<uint32_t*>(xbase);
        float* xs_s = reinterpret_cast<float*>(xbase + Plan::xq_bytes(kc));
        float* xsum_s = reinterpret_cast<float*>(xbase + Plan::xq_bytes(kc) + Plan::xs_bytes(kc));
        const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
        // each warp quantizes exactly the chunks it will consume, four at a time so
        // that their loads overlap
        for (int i0 = 0; i0 < n_my; i0 += 4) {
            float xv[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + u < n_my) {
                    load_x_chunk(xv[u], x, v.k, warp + (i0 + u) * WARPS, lane, aligned);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + u < n_my) {
                    quantize_chunk_to_smem(xv[u], warp + (i0 + u) * WARPS, lane, xq_words, xs_s, xsum_s);
                }
            }
        }
        __syncwarp();
        xsrc.xq = reinterpret_cast<const uint4*>(xq_words);
        xsrc.xs = xs_s;
        xsrc.xsum = xsum_s;
    } else {
        xsrc.xp = xp;
    }

    float acc[NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
        acc[o] = 0.0f;
    }

    // 3. consume tiles as they land; refill each slot right after it has been read
    bool ok = true;
    for (int i = 0; i < n_my; ++i) {
        const int s = i % DEPTH;
        const uint32_t parity = (uint32_t)(i / DEPTH) & 1u;
        if (ok && !mbar_wait(&my_bars[s], parity)) {
            ok = false;
            if (lane == 0) {
                atomicExch(status, 1);
            }
        }
        if (ok) {
            compute_chunk<FMT, MC>(my_slots + (size_t)s * Plan::SLOT, xsrc, warp + i * WARPS, lane, acc);
        }
        __syncwarp();
        if (ok && lane == 0 && i + DEPTH < n_my) {
            fence_proxy_async();  // order this warp's reads of the slot before the refill
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)(warp + (i + DEPTH) * WARPS) * TILE,
                          TILE, &my_bars[s]);
        }
    }

    // 4. partial sums of the warps meet in shared memory
    float* red = reinterpret_cast<float*>(smem + Plan::total(kc, MC) - WARPS * 16 * MC * 4);
    const int g = lane >> 2;
    const int t = lane & 3;
    if constexpr (MC == 1) {
        if (t == 0) {
            red[(warp * 16 + g)] = acc[0];
            red[(warp * 16 + g + 8)] = acc[1];
        }
    } else {
#pragma unroll
        for (int cgi = 0; cgi < Cols<MC>::NCG; ++cgi) {
            red[(warp * 16 + g) * MC + 8 * cgi + 2 * t] = acc[4 * cgi + 0];
            red[(warp * 16 + g) * MC + 8 * cgi + 2 * t + 1] = acc[4 * cgi + 1];
            red[(warp * 16 + g + 8) * MC + 8 * cgi + 2 * t] = acc[4 * cgi + 2];
            red[(warp * 16 + g + 8) * MC + 8 * cgi + 2 * t + 1] = acc[4 * cgi + 3];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * MC; i += WARPS * 32) {
        const int col = i >> 4;
        const int r = i & 15;
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            sum += red[(w * 16 + r) * MC + col];
        }
        const int64_t row = (int64_t)blockIdx.x * 16 + r;
        if (row < v.n && col < m) {
            y[(int64_t)col * v.n + row] = sum;
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
    pdl_launch_dependents();  // the matvec that follows may start fetching its weights
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

    // thread -> (block b, fragment lane)
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

// Ring depth per format: about 36 KB of tiles in flight per CTA.
template <int FMT>
struct Tune {
    static constexpr int WARPS = 4;
    static constexpr int DEPTH = FMT == FMT_Q8_0 ? 2 : FMT == FMT_Q6_K ? 3 : 4;
};

template <int FMT, int MC>
cudaError_t launch_gemv_fmt_mc(const WeightView& w, const float* x, const XPackView& xp, float* y, int m,
                               int* status, cudaStream_t stream)
{
    constexpr int WARPS = Tune<FMT>::WARPS;
    constexpr int DEPTH = Tune<FMT>::DEPTH;
    using Plan = SmemPlan<FMT, WARPS, DEPTH>;
    auto kernel = gemv_kernel<FMT, MC, WARPS, DEPTH>;
    const int smem = Plan::total(w.kc, MC);
    if (smem > 227 * 1024) {
        return cudaErrorInvalidConfiguration;
    }
    // the opt-in limit is a per-device function attribute; raise it only when needed
    static int configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            return e;
        }
        if (dev >= 0 && dev < 64) {
            configured[dev] = smem;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)w.rt);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, w, x, xp, y, m, status);
}

template <int FMT>
cudaError_t launch_gemv_fmt(const WeightView& w, const float* x, const XPackView& xp, float* y, int m, int* status,
                            cudaStream_t stream)
{
    if (m == 1) {
        return launch_gemv_fmt_mc<FMT, 1>(w, x, xp, y, m, status, stream);
    }
    if (m <= 8) {
        return launch_gemv_fmt_mc<FMT, 8>(w, x, xp, y, m, status, stream);
    }
    return launch_gemv_fmt_mc<FMT, 16>(w, x, xp, y, m, status, stream);
}

}  // namespace

cudaError_t launch_pack_x(const float* x, int m, int64_t k, int kc, int cg, const XPackBuffers& out,
                          cudaStream_t stream)
{
    pack_x_kernel<<<dim3(kc, cg), 256, 0, stream>>>(x, m, k, cg, out.xq, out.xs, out.xsum);
    return cudaGetLastError();
}

cudaError_t launch_gemv(const WeightView& w, const float* x, const XPackView& xp, float* y, int m, int* status,
                        cudaStream_t stream)
{
    switch (w.fmt) {
    case FMT_Q4_0: return launch_gemv_fmt<FMT_Q4_0>(w, x, xp, y, m, status, stream);
    case FMT_Q8_0: return launch_gemv_fmt<FMT_Q8_0>(w, x, xp, y, m, status, stream);
    case FMT_Q4_K: return launch_gemv_fmt<FMT_Q4_K>(w, x, xp, y, m, status, stream);
    case FMT_Q6_K: return launch_gemv_fmt<FMT_Q6_K>(w, x, xp, y, m, status, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace qmm

// Device-side building blocks of the dequant-fused matvec, shared by the stand-alone GEMV
// kernels (qmm_gemv.cu) and the persistent decoder kernel (llama_mega.cu): mbarrier / bulk-copy
// PTX wrappers, the integer MMA wrappers, the packed-activation views and the per-chunk
// multiply routines for every block format.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "qmm_common.cuh"

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

// D = A(16x32, row) * B(32x8, col, s8) with a zero C operand.
template <bool A_SIGNED>
__device__ __forceinline__ void mma_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1)
{
    const int z = 0;
    if constexpr (A_SIGNED) {
        asm(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
    } else {
        asm(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
    }
}

// D = A(16x16, row, s8) * B(16x8, col, s8) with a zero C operand.
__device__ __forceinline__ void mma_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    const int z = 0;
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(z));
}

// D = A * B + D  (k32, B s8): second half of a two-MMA block pair.
template <bool A_SIGNED>
__device__ __forceinline__ void mma_k32_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1)
{
    if constexpr (A_SIGNED) {
        asm(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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
//
// B-fragment of one MMA (k32 x 8 columns): column 2r holds the high bytes and column
// 2r+1 the low bytes of activation row 4*j + r of column group j, so lane (g,t) keeps
// in d[0],d[1] the (high, low) sums of weight row g and in d[2],d[3] those of row g+8,
// all for activation row 4*j + t.

// MC = activation rows handled: 1 (only row 0 is live) or a multiple of 4 up to 16.
template <int MC>
struct Cols {
    static constexpr int NCP = MC == 1 ? 1 : MC / 4;  // MMAs (column groups of 4 rows) per block
    static constexpr int NOUT = 2 * NCP;              // accumulators per lane
};

// Batch 1: all compact records (qmm_common.cuh) staged in shared memory.
struct XShared {
    const uint8_t* base;   // [kc] records of XPK1_REC bytes
    const uint8_t* zeros;  // 512 zero bytes for the lanes that carry no activation row
};

// Batches 2..16: the record of one chunk travels with the weight tile into the warp's ring
// slot, behind the tile:  xq [8 blocks][NCP][32 lanes] uint2 | meta [8 blocks][16 rows] int4
template <int NCP>
struct XSlot {
    static constexpr int XQ_BYTES = xpack_xq_bytes(NCP);
    static constexpr int BYTES = xpack_rec_bytes(NCP);
    const uint8_t* base;  // the chunk's record in the current slot
    __device__ __forceinline__ void attach(const uint8_t* p) { base = p; }
    __device__ __forceinline__ uint2 frag(int b, int j, int lane) const
    {
        return *reinterpret_cast<const uint2*>(base + ((b * NCP + j) * 32 + lane) * 8);
    }
    // {8*Q, 128*Q, scale bits, 0} of block b for this lane's activation row 4*j + t
    __device__ __forceinline__ int4 meta(int b, int j, int lane) const
    {
        return *reinterpret_cast<const int4*>(base + XQ_BYTES + (b * 16 + 4 * j + (lane & 3)) * 16);
    }
};

template <int MC>
using XSrc = typename std::conditional<MC == 1, XShared, XSlot<Cols<MC>::NCP>>::type;

// One 16x256 tile, resident in shared memory at `slot`, times the activations of its chunk
// (batches 2..16).  acc[2j], acc[2j+1]: rows g, g+8 for activation row 4j + t.
template <int FMT, int MC>
__device__ __forceinline__ void compute_chunk(const uint8_t* slot, const XSrc<MC>& xs, int lane, float* acc)
{
    constexpr int NCP = Cols<MC>::NCP;
    const int g = lane >> 2;
    int d[4];
    const uint4* qs = reinterpret_cast<const uint4*>(slot) + lane;
    const uint8_t* p1 = slot + tile_p1_offset(FMT);
    const uint8_t* p2 = slot + tile_p2_offset(FMT);

    if constexpr (FMT == FMT_Q4_0) {
        // d[0],d[1]: digit sums of row g over unsigned nibbles n; d[2],d[3]: those of row g+8 over the
        // bytes 16*n(g+8) + n(g), so row g+8 comes out in units of 1/16 after row g's part is removed.
        const uint4 s0 = *reinterpret_cast<const uint4*>(p1 + g * 16);
        const uint4 s1 = *reinterpret_cast<const uint4*>(p1 + (g + 8) * 16);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint4 q = qs[p * 32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w1 = h ? q.z : q.x;  // weights 4t..   rows g | g+8
                const uint32_t w2 = h ? q.w : q.y;  // weights 16+4t..
                const int b = 2 * p + h;
                const float dg = half_of(s0, b);
                const float dg8 = half_of(s1, b) * 0.0625f;
#pragma unroll
                for (int j = 0; j < NCP; ++j) {
                    const uint2 xf = xs.frag(b, j, lane);
                    mma_k32<false>(d, w1 & 0x0F0F0F0Fu, w1, w2 & 0x0F0F0F0Fu, w2, xf.x, xf.y);
                    const int4 mm = xs.meta(b, j, lane);
                    const float xsb = __int_as_float(mm.z);
                    const int vg = d[0] * 256 + d[1];
                    const int vg8 = d[2] * 256 + d[3] - vg;
                    acc[2 * j + 0] = fmaf((float)(vg - mm.x), dg * xsb, acc[2 * j + 0]);
                    acc[2 * j + 1] = fmaf((float)(vg8 - mm.y), dg8 * xsb, acc[2 * j + 1]);
                }
            }
        }
    } else if constexpr (FMT == FMT_Q8_0) {
        const uint4 s0 = *reinterpret_cast<const uint4*>(p1 + g * 16);
        const uint4 s1 = *reinterpret_cast<const uint4*>(p1 + (g + 8) * 16);
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const uint4 q = qs[b * 32];
            const float dg = half_of(s0, b);
            const float dg8 = half_of(s1, b);
#pragma unroll
            for (int j = 0; j < NCP; ++j) {
                const uint2 xf = xs.frag(b, j, lane);
                mma_k32<true>(d, q.x, q.y, q.z, q.w, xf.x, xf.y);
                const float xsb = __int_as_float(xs.meta(b, j, lane).z);
                acc[2 * j + 0] = fmaf((float)(d[0] * 256 + d[1]), dg * xsb, acc[2 * j + 0]);
                acc[2 * j + 1] = fmaf((float)(d[2] * 256 + d[3]), dg8 * xsb, acc[2 * j + 1]);
            }
        }
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
                const uint32_t w1 = h ? q.z : q.x;
                const uint32_t w2 = h ? q.w : q.y;
                const float sg = dd[0] * (float)byte_of_word(scw[0][sb >> 2], sb & 3);
                const float sg8 = dd[1] * (float)byte_of_word(scw[1][sb >> 2], sb & 3) * 0.0625f;
                // "- dmin*m": the same offset on every weight of the sub-block, so it multiplies the
                // sum of the block's quantized activations, (8*Q) / 8
                const float mg = dmin[0] * (float)byte_of_word(mnw[0][sb >> 2], sb & 3) * 0.125f;
                const float mg8 = dmin[1] * (float)byte_of_word(mnw[1][sb >> 2], sb & 3) * 0.125f;
#pragma unroll
                for (int j = 0; j < NCP; ++j) {
                    const uint2 xf = xs.frag(sb, j, lane);
                    mma_k32<false>(d, w1 & 0x0F0F0F0Fu, w1, w2 & 0x0F0F0F0Fu, w2, xf.x, xf.y);
                    const int4 mm = xs.meta(sb, j, lane);
                    const float xsb = __int_as_float(mm.z);
                    const int vg = d[0] * 256 + d[1];
                    const int vg8 = d[2] * 256 + d[3] - vg;
                    const float q8 = (float)mm.x * xsb;
                    acc[2 * j + 0] = fmaf((float)vg, sg * xsb, fmaf(-mg, q8, acc[2 * j + 0]));
                    acc[2 * j + 1] = fmaf((float)vg8, sg8 * xsb, fmaf(-mg8, q8, acc[2 * j + 1]));
                }
            }
        }
    } else {  // Q6_K: A byte = 4 * (q - 32) as int8, one k16 MMA per 16-wide sub-block
        const uint4 s0 = *reinterpret_cast<const uint4*>(p1 + g * 16);
        const uint4 s1 = *reinterpret_cast<const uint4*>(p1 + (g + 8) * 16);
        const float dg = __half2float(*reinterpret_cast<const __half*>(p2 + g * 2)) * 0.25f;
        const float dg8 = __half2float(*reinterpret_cast<const __half*>(p2 + (g + 8) * 2)) * 0.25f;
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
            for (int j = 0; j < NCP; ++j) {
                const uint2 xf0 = xs.frag(2 * quad, j, lane);
                const uint2 xf1 = xs.frag(2 * quad + 1, j, lane);
                const float xsb0 = __int_as_float(xs.meta(2 * quad, j, lane).z);
                const float xsb1 = __int_as_float(xs.meta(2 * quad + 1, j, lane).z);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int sb = 4 * quad + jj;
                    const uint2& xf = (jj >> 1) ? xf1 : xf0;
                    const float xsb = (jj >> 1) ? xsb1 : xsb0;
                    mma_k16(d, out[0][jj], out[1][jj], (jj & 1) ? xf.y : xf.x);
                    const float sg = dg * (float)(int)(signed char)byte_of(s0, sb);
                    const float sg8 = dg8 * (float)(int)(signed char)byte_of(s1, sb);
                    acc[2 * j + 0] = fmaf((float)(d[0] * 256 + d[1]), sg * xsb, acc[2 * j + 0]);
                    acc[2 * j + 1] = fmaf((float)(d[2] * 256 + d[3]), sg8 * xsb, acc[2 * j + 1]);
                }
            }
        }
    }
}

// ---- batch 1 ---------------------------------------------------------------------------------
//
// With one activation row only columns 0 and 1 of an MMA would be live and the scalar
// work that follows it (combine the two digits, convert, scale) would run with three
// quarters of the lanes idle.  So two neighbouring blocks share an MMA instead: the A
// operand takes k-slots 0..15 from block b and k-slots 16..31 from block b+1 (for a
// fragment that is only a choice of registers), the B operand is block diagonal —
// columns 0,1 carry the digits of block b's activations in k-slots 0..15, columns 2,3
// those of block b+1 in k-slots 16..31 — and a second MMA adds the other halves of
// both blocks.  Lane t=0 then folds block b and lane t=1 block b+1 at the same time.

template <int FMT>
__device__ __forceinline__ void compute_chunk_m1(const uint8_t* slot, const XShared& xs, int c, int lane, float* acc)
{
    const int g = lane >> 2;
    const int t = lane & 3;
    const int tsel = t & 1;
    const uint8_t* rec = xs.base + (size_t)c * XPK1_REC;
    // Per-lane sources of the B registers: lanes g<2 feed b0 (columns 0,1 = digits of the
    // first block of a pair), lanes g in {2,3} feed b1 (columns 2,3 = second block); every
    // other register comes from the zero page.  Entry = uint2 {weights 4t.., weights 16+4t..}.
    const uint8_t* xrow = rec + ((g & 1) * 4 + t) * 8;
    const uint8_t* b0p = g < 2 ? xrow : xs.zeros;
    const uint8_t* b1p = (g >> 1) == 1 ? xrow + 64 : xs.zeros;
    const int4* meta = reinterpret_cast<const int4*>(rec + XPK1_META);
    const uint4* qs = reinterpret_cast<const uint4*>(slot) + lane;
    const uint8_t* p1 = slot + tile_p1_offset(FMT);
    const uint8_t* p2 = slot + tile_p2_offset(FMT);
    float a0 = 0.0f, a1 = 0.0f;
    int d[4];

    if constexpr (FMT == FMT_Q4_0) {
        const __half* dg_p = reinterpret_cast<const __half*>(p1 + g * 16) + tsel;
        const __half* dg8_p = reinterpret_cast<const __half*>(p1 + (g + 8) * 16) + tsel;
#ifndef QMM_M1_BATCH
#define QMM_M1_BATCH 1
#endif
        // every shared-memory load of QMM_M1_BATCH block pairs is issued before the first MMA of the batch
#pragma unroll
        for (int p0 = 0; p0 < 4; p0 += QMM_M1_BATCH) {
            uint2 x0[QMM_M1_BATCH], x1[QMM_M1_BATCH];
            uint4 q[QMM_M1_BATCH];
            int4 mm[QMM_M1_BATCH];
            float dg[QMM_M1_BATCH], dg8[QMM_M1_BATCH];
#pragma unroll
            for (int i = 0; i < QMM_M1_BATCH; ++i) {
                const int p = p0 + i;
                x0[i] = *reinterpret_cast<const uint2*>(b0p + p * 128);
                x1[i] = *reinterpret_cast<const uint2*>(b1p + p * 128);
                q[i] = qs[p * 32];  // {blk 2p w 4t.., blk 2p w 16+4t.., blk 2p+1 w 4t.., blk 2p+1 w 16+4t..}
                mm[i] = meta[2 * p + tsel];
                dg[i] = __half2float(dg_p[2 * p]);
                dg8[i] = __half2float(dg8_p[2 * p]);
            }
#pragma unroll
            for (int i = 0; i < QMM_M1_BATCH; ++i) {
                mma_k32<false>(d, q[i].x & 0x0F0F0F0Fu, q[i].x, q[i].z & 0x0F0F0F0Fu, q[i].z, x0[i].x, x1[i].x);
                mma_k32_acc<false>(d, q[i].y & 0x0F0F0F0Fu, q[i].y, q[i].w & 0x0F0F0F0Fu, q[i].w, x0[i].y, x1[i].y);
                const float xsb = __int_as_float(mm[i].z);
                const int vg = d[0] * 256 + d[1];
                const int vg8 = d[2] * 256 + d[3] - vg;
                a0 = fmaf((float)(vg - mm[i].x), dg[i] * xsb, a0);
                a1 = fmaf((float)(vg8 - mm[i].y), dg8[i] * xsb, a1);
            }
        }
        acc[0] += a0;
        acc[1] = fmaf(a1, 0.0625f, acc[1]);
    } else if constexpr (FMT == FMT_Q8_0) {
        const __half* dg_p = reinterpret_cast<const __half*>(p1 + g * 16) + tsel;
        const __half* dg8_p = reinterpret_cast<const __half*>(p1 + (g + 8) * 16) + tsel;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint2 x0 = *reinterpret_cast<const uint2*>(b0p + p * 128);
            const uint2 x1 = *reinterpret_cast<const uint2*>(b1p + p * 128);
            const uint4 qa = qs[(2 * p) * 32];
            const uint4 qb = qs[(2 * p + 1) * 32];
            mma_k32<true>(d, qa.x, qa.y, qb.x, qb.y, x0.x, x1.x);
            mma_k32_acc<true>(d, qa.z, qa.w, qb.z, qb.w, x0.y, x1.y);
            const float xsb = __int_as_float(meta[2 * p + tsel].z);
            a0 = fmaf((float)(d[0] * 256 + d[1]), __half2float(dg_p[2 * p]) * xsb, a0);
            a1 = fmaf((float)(d[2] * 256 + d[3]), __half2float(dg8_p[2 * p]) * xsb, a1);
        }
        acc[0] += a0;
        acc[1] += a1;
    } else if constexpr (FMT == FMT_Q4_K) {
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
        float m0 = 0.0f, m1 = 0.0f;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint2 x0 = *reinterpret_cast<const uint2*>(b0p + p * 128);
            const uint2 x1 = *reinterpret_cast<const uint2*>(b1p + p * 128);
            const uint4 q = qs[p * 32];
            mma_k32<false>(d, q.x & 0x0F0F0F0Fu, q.x, q.z & 0x0F0F0F0Fu, q.z, x0.x, x1.x);
            mma_k32_acc<false>(d, q.y & 0x0F0F0F0Fu, q.y, q.w & 0x0F0F0F0Fu, q.w, x0.y, x1.y);
            // this lane's sub-block is 2p + tsel: byte (2p & 3) + tsel of word p >> 1
            const int sh = 8 * ((2 * p) & 3) + 8 * tsel;
            const int4 mm = meta[2 * p + tsel];
            const float xsb = __int_as_float(mm.z);
            const float sg = dd[0] * (float)((scw[0][p >> 1] >> sh) & 0xFFu);
            const float sg8 = dd[1] * (float)((scw[1][p >> 1] >> sh) & 0xFFu);
            const float mg = dmin[0] * (float)((mnw[0][p >> 1] >> sh) & 0xFFu);
            const float mg8 = dmin[1] * (float)((mnw[1][p >> 1] >> sh) & 0xFFu);
            const int vg = d[0] * 256 + d[1];
            const int vg8 = d[2] * 256 + d[3] - vg;
            a0 = fmaf((float)vg, sg * xsb, a0);
            a1 = fmaf((float)vg8, sg8 * xsb, a1);
            const float q8 = (float)mm.x * xsb;  // 8 * sum of the block's activations, in their own units
            m0 = fmaf(mg, q8, m0);
            m1 = fmaf(mg8, q8, m1);
        }
        acc[0] += fmaf(-m0, 0.125f, a0);
        acc[1] += fmaf(-m1, 0.125f, a1 * 0.0625f);
    } else {  // Q6_K: the two 16-wide sub-blocks of a 32-block share one k32 MMA
        const float dg = __half2float(*reinterpret_cast<const __half*>(p2 + g * 2));
        const float dg8 = __half2float(*reinterpret_cast<const __half*>(p2 + (g + 8) * 2));
        const signed char* sc_g = reinterpret_cast<const signed char*>(p1 + g * 16) + tsel;
        const signed char* sc_g8 = reinterpret_cast<const signed char*>(p1 + (g + 8) * 16) + tsel;
        // for Q6_K the pair is (sub-block 2b, 2b+1) of ONE 32-block b: lanes g<2 supply the
        // first word (weights 4t..) as b0, lanes g in {2,3} the second (weights 16+4t..) as b1
        const uint8_t* c0p = g < 2 ? xrow : xs.zeros;
        const uint8_t* c1p = (g >> 1) == 1 ? xrow + 4 : xs.zeros;
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
            for (int hb = 0; hb < 2; ++hb) {
                const int b = 2 * quad + hb;  // 32-block, sub-blocks 2b and 2b+1
                const uint32_t xb0 = *reinterpret_cast<const uint32_t*>(c0p + b * 64);
                const uint32_t xb1 = *reinterpret_cast<const uint32_t*>(c1p + b * 64);
                mma_k32<true>(d, out[0][2 * hb], out[1][2 * hb], out[0][2 * hb + 1], out[1][2 * hb + 1], xb0, xb1);
                const float xsb = __int_as_float(meta[b].z);
                const float sg = dg * (float)(int)sc_g[2 * b];
                const float sg8 = dg8 * (float)(int)sc_g8[2 * b];
                a0 = fmaf((float)(d[0] * 256 + d[1]), sg * xsb, a0);
                a1 = fmaf((float)(d[2] * 256 + d[3]), sg8 * xsb, a1);
            }
        }
        acc[0] = fmaf(a0, 0.25f, acc[0]);
        acc[1] = fmaf(a1, 0.25f, acc[1]);
    }
}

}  // namespace
}  // namespace qmm

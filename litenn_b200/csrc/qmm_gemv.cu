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
// The activations are quantized once per call by pack_x_kernel (16 bits per value,
// scale per (row, 256 chunk)) and stored in B-fragment order with the signed high
// and signed low byte of one activation row in adjacent MMA columns, so one MMA
// yields both partial sums of four activation rows and they meet in one lane.
// Batch 1 brings its packed activations into shared memory with one more bulk copy;
// batches 2..16 read them through L1.  Kernels are launched with programmatic
// dependent launch: the weight copies are issued before griddepcontrol.wait, so in
// a chain of dependent matvecs the next kernel's weights stream while the previous
// kernel drains.
#include <cstdlib>

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

// Batch 1: packed activations staged in shared memory (compact: only lanes 0..7 hold data).
//   xq   [kc][8 blocks][8 lanes] uint2;  xs [kc];  xsum [kc][8]
struct XShared {
    const uint8_t* xq;
    const float* xs;
    const int2* xsum;      // {8*Q, 128*Q} per block
    const uint8_t* zeros;  // 512 zero bytes for the lanes that carry no activation row
    const uint8_t* cur;    // per-lane base for the current chunk
    __device__ __forceinline__ void begin_chunk(int c, int lane)
    {
        cur = lane < 8 ? xq + (size_t)c * 512 + lane * 8 : zeros + (lane & 7) * 8;
    }
    __device__ __forceinline__ uint2 frag(int /*c*/, int b, int /*j*/, int /*lane*/) const
    {
        return *reinterpret_cast<const uint2*>(cur + b * 64);
    }
    __device__ __forceinline__ float scale(int c, int /*j*/, int /*lane*/) const { return xs[c]; }
    __device__ __forceinline__ int2 bsum(int c, int b, int /*j*/, int /*lane*/) const { return xsum[c * 8 + b]; }
};

// Batches 2..16: packed activations read from global memory (L1-resident).
//   xq [kc][8 blocks][ncp][32 lanes] uint2;  xs [kc][16];  xsum [kc][8][16] int2
struct XGlobal {
    const uint2* xq;
    const float* xs;
    const int2* xsum;
    int ncp;
    __device__ __forceinline__ void begin_chunk(int, int) {}
    __device__ __forceinline__ uint2 frag(int c, int b, int j, int lane) const
    {
        return __ldg(xq + ((size_t)(c * 8 + b) * ncp + j) * 32 + lane);
    }
    __device__ __forceinline__ float scale(int c, int j, int lane) const
    {
        return __ldg(xs + c * 16 + 4 * j + (lane & 3));
    }
    __device__ __forceinline__ int2 bsum(int c, int b, int j, int lane) const
    {
        return __ldg(xsum + (size_t)(c * 8 + b) * 16 + 4 * j + (lane & 3));
    }
};

template <int MC>
using XSrc = typename std::conditional<MC == 1, XShared, XGlobal>::type;

// accc += (256*hi + lo) * row scale
__device__ __forceinline__ void fold(float* accc, int j, const int (&d)[4], float sg, float sg8)
{
    accc[2 * j + 0] = fmaf((float)(d[0] * 256 + d[1]), sg, accc[2 * j + 0]);
    accc[2 * j + 1] = fmaf((float)(d[2] * 256 + d[3]), sg8, accc[2 * j + 1]);
}

// 4-bit formats: d[0],d[1] are the digit sums of row g over unsigned nibbles n, d[2],d[3]
// those of row g+8 over the bytes 16*n(g+8) + n(g).  `off` is what turns n into the
// signed quant (8*Q for Q4_0, 0 for Q4_K), `off16` the same for row g+8 in units of 1/16.
__device__ __forceinline__ void fold4(float* accc, int j, const int (&d)[4], float sg, float sg8, int off, int off16)
{
    const int vg = d[0] * 256 + d[1];
    const int vg8 = d[2] * 256 + d[3] - vg;
    accc[2 * j + 0] = fmaf((float)(vg - off), sg, accc[2 * j + 0]);
    accc[2 * j + 1] = fmaf((float)(vg8 - off16), sg8, accc[2 * j + 1]);
}

// acc += accc * (activation scale of the chunk) * extra
template <int MC>
__device__ __forceinline__ void fold_chunk(float* acc, const float* accc, const XSrc<MC>& xs, int c, int lane,
                                           float extra)
{
#pragma unroll
    for (int j = 0; j < Cols<MC>::NCP; ++j) {
        const float sx = xs.scale(c, j, lane) * extra;
        acc[2 * j + 0] = fmaf(accc[2 * j + 0], sx, acc[2 * j + 0]);
        acc[2 * j + 1] = fmaf(accc[2 * j + 1], sx, acc[2 * j + 1]);
    }
}

// Same, when row g+8 was accumulated in units of 1/16 (4-bit formats).
template <int MC>
__device__ __forceinline__ void fold_chunk4(float* acc, const float* accc, const XSrc<MC>& xs, int c, int lane)
{
#pragma unroll
    for (int j = 0; j < Cols<MC>::NCP; ++j) {
        const float sx = xs.scale(c, j, lane);
        acc[2 * j + 0] = fmaf(accc[2 * j + 0], sx, acc[2 * j + 0]);
        acc[2 * j + 1] = fmaf(accc[2 * j + 1], sx * 0.0625f, acc[2 * j + 1]);
    }
}

// One 16x256 tile, resident in shared memory at `slot`, times the activations of chunk c.
template <int FMT, int MC>
__device__ __forceinline__ void compute_chunk(const uint8_t* slot, XSrc<MC>& xs, int c, int lane, float* acc)
{
    constexpr int NCP = Cols<MC>::NCP;
    constexpr int NOUT = Cols<MC>::NOUT;
    const int g = lane >> 2;
    float accc[NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
        accc[o] = 0.0f;
    }
    int d[4];
    const uint4* qs = reinterpret_cast<const uint4*>(slot) + lane;
    const uint8_t* p1 = slot + tile_p1_offset(FMT);
    const uint8_t* p2 = slot + tile_p2_offset(FMT);
    xs.begin_chunk(c, lane);

    if constexpr (FMT == FMT_Q4_0) {
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
                const float dg8 = half_of(s1, b);
#pragma unroll
                for (int j = 0; j < NCP; ++j) {
                    const uint2 xf = xs.frag(c, b, j, lane);
                    mma_k32<false>(d, w1 & 0x0F0F0F0Fu, w1, w2 & 0x0F0F0F0Fu, w2, xf.x, xf.y);
                    const int2 Q = xs.bsum(c, b, j, lane);
                    fold4(accc, j, d, dg, dg8, Q.x, Q.y);
                }
            }
        }
        fold_chunk4<MC>(acc, accc, xs, c, lane);
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
                const uint2 xf = xs.frag(c, b, j, lane);
                mma_k32<true>(d, q.x, q.y, q.z, q.w, xf.x, xf.y);
                fold(accc, j, d, dg, dg8);
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
        float macc[NOUT];
#pragma unroll
        for (int o = 0; o < NOUT; ++o) {
            macc[o] = 0.0f;
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
                const float sg8 = dd[1] * (float)byte_of_word(scw[1][sb >> 2], sb & 3);
                const float mg = dmin[0] * (float)byte_of_word(mnw[0][sb >> 2], sb & 3);
                const float mg8 = dmin[1] * (float)byte_of_word(mnw[1][sb >> 2], sb & 3);
#pragma unroll
                for (int j = 0; j < NCP; ++j) {
                    const uint2 xf = xs.frag(c, sb, j, lane);
                    mma_k32<false>(d, w1 & 0x0F0F0F0Fu, w1, w2 & 0x0F0F0F0Fu, w2, xf.x, xf.y);
                    fold4(accc, j, d, sg, sg8, 0, 0);
                    // "- dmin*m": the same offset on every weight of the block, so it
                    // multiplies the sum of the block's (quantized) activations, 8*Q / 8
                    const float qs8 = (float)xs.bsum(c, sb, j, lane).x;
                    macc[2 * j + 0] = fmaf(mg, qs8, macc[2 * j + 0]);
                    macc[2 * j + 1] = fmaf(mg8, qs8, macc[2 * j + 1]);
                }
            }
        }
        fold_chunk4<MC>(acc, accc, xs, c, lane);
#pragma unroll
        for (int j = 0; j < NCP; ++j) {
            const float sx = xs.scale(c, j, lane) * 0.125f;
            acc[2 * j + 0] = fmaf(-macc[2 * j + 0], sx, acc[2 * j + 0]);
            acc[2 * j + 1] = fmaf(-macc[2 * j + 1], sx, acc[2 * j + 1]);
        }
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
            for (int j = 0; j < NCP; ++j) {
                const uint2 xf0 = xs.frag(c, 2 * quad, j, lane);
                const uint2 xf1 = xs.frag(c, 2 * quad + 1, j, lane);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int sb = 4 * quad + jj;
                    const uint2& xf = (jj >> 1) ? xf1 : xf0;
                    mma_k16(d, out[0][jj], out[1][jj], (jj & 1) ? xf.y : xf.x);
                    const float sg = dg * (float)(int)(signed char)byte_of(s0, sb);
                    const float sg8 = dg8 * (float)(int)(signed char)byte_of(s1, sb);
                    fold(accc, j, d, sg, sg8);
                }
            }
        }
        fold_chunk<MC>(acc, accc, xs, c, lane, 0.25f);
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
    // Per-lane sources of the B registers: lanes g<2 feed b0 (columns 0,1 = digits of the
    // first block of a pair), lanes g in {2,3} feed b1 (columns 2,3 = second block); every
    // other register comes from the zero page.  Entry = uint2 {weights 4t.., weights 16+4t..}.
    const uint8_t* xrow = xs.xq + (size_t)c * 512 + ((g & 1) * 4 + t) * 8;
    const uint8_t* b0p = g < 2 ? xrow : xs.zeros;
    const uint8_t* b1p = (g >> 1) == 1 ? xrow + 64 : xs.zeros;
    const uint4* qs = reinterpret_cast<const uint4*>(slot) + lane;
    const uint8_t* p1 = slot + tile_p1_offset(FMT);
    const uint8_t* p2 = slot + tile_p2_offset(FMT);
    float accc0 = 0.0f, accc1 = 0.0f;
    int d[4];

    if constexpr (FMT == FMT_Q4_0) {
        const __half* dg_p = reinterpret_cast<const __half*>(p1 + g * 16) + tsel;
        const __half* dg8_p = reinterpret_cast<const __half*>(p1 + (g + 8) * 16) + tsel;
        const int2* qsum = xs.xsum + c * 8 + tsel;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint2 x0 = *reinterpret_cast<const uint2*>(b0p + p * 128);
            const uint2 x1 = *reinterpret_cast<const uint2*>(b1p + p * 128);
            const uint4 q = qs[p * 32];  // {blk 2p w 4t.., blk 2p w 16+4t.., blk 2p+1 w 4t.., blk 2p+1 w 16+4t..}
            mma_k32<false>(d, q.x & 0x0F0F0F0Fu, q.x, q.z & 0x0F0F0F0Fu, q.z, x0.x, x1.x);
            mma_k32_acc<false>(d, q.y & 0x0F0F0F0Fu, q.y, q.w & 0x0F0F0F0Fu, q.w, x0.y, x1.y);
            const int2 Q = qsum[2 * p];
            const int vg = d[0] * 256 + d[1];
            const int vg8 = d[2] * 256 + d[3] - vg;
            accc0 = fmaf((float)(vg - Q.x), __half2float(dg_p[2 * p]), accc0);
            accc1 = fmaf((float)(vg8 - Q.y), __half2float(dg8_p[2 * p]), accc1);
        }
        const float sx = xs.xs[c];
        acc[0] = fmaf(accc0, sx, acc[0]);
        acc[1] = fmaf(accc1, sx * 0.0625f, acc[1]);
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
            accc0 = fmaf((float)(d[0] * 256 + d[1]), __half2float(dg_p[2 * p]), accc0);
            accc1 = fmaf((float)(d[2] * 256 + d[3]), __half2float(dg8_p[2 * p]), accc1);
        }
        const float sx = xs.xs[c];
        acc[0] = fmaf(accc0, sx, acc[0]);
        acc[1] = fmaf(accc1, sx, acc[1]);
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
        const int2* qsum = xs.xsum + c * 8 + tsel;
        float macc0 = 0.0f, macc1 = 0.0f;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint2 x0 = *reinterpret_cast<const uint2*>(b0p + p * 128);
            const uint2 x1 = *reinterpret_cast<const uint2*>(b1p + p * 128);
            const uint4 q = qs[p * 32];
            mma_k32<false>(d, q.x & 0x0F0F0F0Fu, q.x, q.z & 0x0F0F0F0Fu, q.z, x0.x, x1.x);
            mma_k32_acc<false>(d, q.y & 0x0F0F0F0Fu, q.y, q.w & 0x0F0F0F0Fu, q.w, x0.y, x1.y);
            // this lane's sub-block is 2p + tsel: byte (2p & 3) + tsel of word p >> 1
            const int sh = 8 * ((2 * p) & 3) + 8 * tsel;
            const float sg = dd[0] * (float)((scw[0][p >> 1] >> sh) & 0xFFu);
            const float sg8 = dd[1] * (float)((scw[1][p >> 1] >> sh) & 0xFFu);
            const float mg = dmin[0] * (float)((mnw[0][p >> 1] >> sh) & 0xFFu);
            const float mg8 = dmin[1] * (float)((mnw[1][p >> 1] >> sh) & 0xFFu);
            const int vg = d[0] * 256 + d[1];
            const int vg8 = d[2] * 256 + d[3] - vg;
            accc0 = fmaf((float)vg, sg, accc0);
            accc1 = fmaf((float)vg8, sg8, accc1);
            const float qs8 = (float)qsum[2 * p].x;  // 8 * sum of the block's quantized activations
            macc0 = fmaf(mg, qs8, macc0);
            macc1 = fmaf(mg8, qs8, macc1);
        }
        const float sx = xs.xs[c];
        acc[0] = fmaf(accc0, sx, fmaf(-macc0, sx * 0.125f, acc[0]));
        acc[1] = fmaf(accc1, sx * 0.0625f, fmaf(-macc1, sx * 0.125f, acc[1]));
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
                const float sg = dg * (float)(int)sc_g[2 * b];
                const float sg8 = dg8 * (float)(int)sc_g8[2 * b];
                accc0 = fmaf((float)(d[0] * 256 + d[1]), sg, accc0);
                accc1 = fmaf((float)(d[2] * 256 + d[3]), sg8, accc1);
            }
        }
        const float sx = xs.xs[c] * 0.25f;
        acc[0] = fmaf(accc0, sx, acc[0]);
        acc[1] = fmaf(accc1, sx, acc[1]);
    }
}

// ---- the kernel -----------------------------------------------------------------------------

#ifdef QMM_TRACE
// Development-only timeline capture (built with -DQMM_TRACE, never in the product library).
__device__ unsigned long long* g_trace_buf = nullptr;
__device__ unsigned int g_trace_cursor = 0;
__device__ unsigned int g_trace_cap = 0;
__device__ __forceinline__ unsigned long long gtime()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define QMM_TP(i)                  \
    do {                           \
        if (threadIdx.x == 0) {    \
            tp_g[i] = gtime();     \
            tp_c[i] = clock64();   \
        }                          \
    } while (0)
#else
#define QMM_TP(i) \
    do {          \
    } while (0)
#endif

// Shared memory of one CTA, carved from the dynamic allocation:
//   slots  WARPS*DEPTH tiles | mbarriers (+1 for the activations) | (batch 1) packed
//   activations + 512 zero bytes | cross-warp reduction
template <int FMT, int WARPS, int DEPTH>
struct SmemPlan {
    static constexpr int SLOT = tile_bytes(FMT);
    static constexpr int SLOTS_BYTES = WARPS * DEPTH * SLOT;
    static constexpr int BAR_OFF = SLOTS_BYTES;
    static constexpr int BAR_BYTES = (((WARPS * DEPTH + 1) * 8 + 15) / 16) * 16;
    static constexpr int X_OFF = BAR_OFF + BAR_BYTES;
    __host__ __device__ static int x_bytes(int kc, int mc) { return mc == 1 ? (int)xpack1_bytes(kc) + 512 : 0; }
    __host__ __device__ static int red_off(int kc, int mc) { return X_OFF + x_bytes(kc, mc); }
    __host__ __device__ static int total(int kc, int mc) { return red_off(kc, mc) + WARPS * 16 * mc * 4; }
};

template <int FMT, int MC, int WARPS, int DEPTH>
__global__ void __launch_bounds__(WARPS * 32)
    gemv_kernel(WeightView v, XPackView xp, float* __restrict__ y, int m, int* __restrict__ status)
{
    using Plan = SmemPlan<FMT, WARPS, DEPTH>;
    constexpr int NOUT = Cols<MC>::NOUT;
    constexpr uint32_t TILE = tile_bytes(FMT);
    extern __shared__ __align__(128) uint8_t smem[];

#ifdef QMM_TRACE
    unsigned long long tp_g[6] = {}, tp_c[6] = {};
#endif
    QMM_TP(0);
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int kc = v.kc;
    uint8_t* my_slots = smem + (size_t)warp * DEPTH * Plan::SLOT;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFF);
    uint64_t* my_bars = bars + warp * DEPTH;
    uint64_t* xbar = bars + WARPS * DEPTH;
    const uint8_t* my_tiles = v.tiles + (size_t)blockIdx.x * kc * TILE;
    const int n_my = warp < kc ? (kc - warp + WARPS - 1) / WARPS : 0;

    // 1. start the weight stream: the first DEPTH tiles of this warp
    if (lane == 0) {
        for (int s = 0; s < DEPTH; ++s) {
            mbar_init(&my_bars[s], 1);
        }
        if (warp == 0) {
            mbar_init(xbar, 1);
        }
        fence_barrier_init();
        for (int s = 0; s < DEPTH && s < n_my; ++s) {
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)(warp + s * WARPS) * TILE, TILE,
                          &my_bars[s]);
        }
    }
    if constexpr (MC == 1) {
        // zero page for the lanes that carry no activation row
        uint32_t* z = reinterpret_cast<uint32_t*>(smem + Plan::X_OFF + xpack1_bytes(kc));
        if (threadIdx.x < 128) {
            z[threadIdx.x] = 0u;
        }
    }
    pdl_launch_dependents();
    // 2. everything below may read what the previous kernel in the stream produced
    pdl_wait();
    QMM_TP(1);

    XSrc<MC> xsrc;
    bool ok = true;
    if constexpr (MC == 1) {
        uint8_t* xbase = smem + Plan::X_OFF;
        const uint32_t xbytes = (uint32_t)xpack1_bytes(kc);
        if (threadIdx.x == 0) {  // the thread that initialised xbar
            mbar_expect_tx(xbar, xbytes);
            bulk_copy_g2s(xbase, xp.xq, xbytes, xbar);
        }
        __syncthreads();  // xbar initialised, zero page written
        xsrc.xq = xbase;
        xsrc.xs = reinterpret_cast<const float*>(xbase + xpack1_xs_offset(kc));
        xsrc.xsum = reinterpret_cast<const int2*>(xbase + xpack1_xsum_offset(kc));
        xsrc.zeros = xbase + xbytes;
        xsrc.cur = xbase;
        if (!mbar_wait(xbar, 0)) {
            ok = false;
            if (lane == 0) {
                atomicExch(status, 2);
            }
        }
    } else {
        xsrc.xq = reinterpret_cast<const uint2*>(xp.xq);
        xsrc.xs = xp.xs;
        xsrc.xsum = xp.xsum;
        xsrc.ncp = xp.ncp;
    }

    QMM_TP(2);
    float acc[NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
        acc[o] = 0.0f;
    }

    // 3. consume tiles as they land; refill each slot right after it has been read
    for (int i = 0; i < n_my; ++i) {
        const int s = i % DEPTH;
        const uint32_t parity = (uint32_t)(i / DEPTH) & 1u;
        if (ok && !mbar_wait(&my_bars[s], parity)) {
            ok = false;
            if (lane == 0) {
                atomicExch(status, 1);
            }
        }
#ifdef QMM_TRACE
        if (i == 0) {
            QMM_TP(3);
        }
#endif
        if (ok) {
            if constexpr (MC == 1) {
                compute_chunk_m1<FMT>(my_slots + (size_t)s * Plan::SLOT, xsrc, warp + i * WARPS, lane, acc);
            } else {
                compute_chunk<FMT, MC>(my_slots + (size_t)s * Plan::SLOT, xsrc, warp + i * WARPS, lane, acc);
            }
        }
        __syncwarp();
        if (ok && lane == 0 && i + DEPTH < n_my) {
            fence_proxy_async();  // order this warp's reads of the slot before the refill
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)(warp + (i + DEPTH) * WARPS) * TILE,
                          TILE, &my_bars[s]);
        }
    }

    QMM_TP(4);
    // 4. partial sums of the warps meet in shared memory: red[warp][row][activation row]
    float* red = reinterpret_cast<float*>(smem + Plan::red_off(kc, MC));
    const int g = lane >> 2;
    const int t = lane & 3;
    if constexpr (MC == 1) {
        // lanes t=0 and t=1 each folded one block of every pair
        acc[0] += __shfl_xor_sync(0xFFFFFFFFu, acc[0], 1);
        acc[1] += __shfl_xor_sync(0xFFFFFFFFu, acc[1], 1);
        if (t == 0) {
            red[warp * 16 + g] = acc[0];
            red[warp * 16 + g + 8] = acc[1];
        }
    } else {
#pragma unroll
        for (int j = 0; j < Cols<MC>::NCP; ++j) {
            red[(warp * 16 + g) * MC + 4 * j + t] = acc[2 * j + 0];
            red[(warp * 16 + g + 8) * MC + 4 * j + t] = acc[2 * j + 1];
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
#ifdef QMM_TRACE
    QMM_TP(5);
    if (threadIdx.x == 0 && g_trace_buf != nullptr) {
        const unsigned int slot = atomicAdd(&g_trace_cursor, 1u);
        if (slot < g_trace_cap) {
            unsigned long long* r = g_trace_buf + (size_t)slot * 16;
            unsigned int smid;
            asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
            r[0] = reinterpret_cast<unsigned long long>(v.tiles);
            r[1] = ((unsigned long long)smid << 32) | blockIdx.x;
            for (int i = 0; i < 6; ++i) {
                r[2 + i] = tp_g[i];
                r[8 + i] = tp_c[i];
            }
        }
    }
#endif
}

// ---- batch 1, persistent and statically balanced ---------------------------------------------
//
// The tiles of a weight are one linear array ([row tile][chunk]); unit u = tile u.
// CTA j of G takes the contiguous run [U*j/G, U*(j+1)/G) and warp w of the CTA the
// w-th of W equal parts of that run, so every SM streams the same number of bytes
// (to within one tile) and each warp reads one contiguous byte range through its own
// ring of DEPTH slots.  A warp keeps two fp32 sums per lane while it stays inside one
// row tile and parks them in shared memory when the row tile changes; at the end the
// CTA adds the parked sums per row tile in a fixed order.  A row tile that straddles
// CTAs is finished by the CTA that holds its last unit: the others publish their part
// through `scratch` (16 floats per CTA) and a flag, the owner waits for the flags of
// its left neighbours with a bounded spin and adds the parts in a fixed order, so the
// result does not depend on timing.  Lower-numbered CTAs start first, and a CTA only
// ever waits for lower-numbered ones, so the wait cannot deadlock.
struct StreamKArgs {
    float* scratch;        // [grid][16]
    unsigned int* flags;   // [grid], zero between launches
};

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_u32(unsigned int* p, unsigned int v)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int FMT, int WARPS, int DEPTH>
struct StreamKPlan {
    static constexpr int SLOT = tile_bytes(FMT);
    static constexpr int SLOTS_BYTES = WARPS * DEPTH * SLOT;
    static constexpr int BAR_OFF = SLOTS_BYTES;
    static constexpr int BAR_BYTES = (((WARPS * DEPTH + 1) * 8 + 15) / 16) * 16;
    static constexpr int X_OFF = BAR_OFF + BAR_BYTES;
    __host__ __device__ static int x_bytes(int kc) { return (int)xpack1_bytes(kc) + 512; }
    __host__ __device__ static int table_off(int kc) { return X_OFF + x_bytes(kc); }
    // row tiles one CTA can touch: a run of `len` units crosses at most len/kc + 2 of them
    __host__ __device__ static int max_rt(long long units_per_cta, int kc) { return (int)(units_per_cta / kc) + 2; }
    __host__ __device__ static int total(int kc, long long units_per_cta)
    {
        return table_off(kc) + max_rt(units_per_cta, kc) * WARPS * 16 * 4;
    }
};

template <int FMT, int WARPS, int DEPTH>
__global__ void __launch_bounds__(WARPS * 32, 1)
    gemv_m1_streamk_kernel(WeightView v, XPackView xp, float* __restrict__ y, StreamKArgs sk, int* __restrict__ status)
{
    using Plan = StreamKPlan<FMT, WARPS, DEPTH>;
    constexpr uint32_t TILE = tile_bytes(FMT);
    extern __shared__ __align__(128) uint8_t smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int kc = v.kc;
    const long long U = (long long)v.rt * kc;
    const long long G = gridDim.x;
    const long long j = blockIdx.x;
    const long long u0 = U * j / G;
    const long long u1 = U * (j + 1) / G;
    const long long len = u1 - u0;
    const long long w0 = u0 + len * warp / WARPS;
    const long long w1 = u0 + len * (warp + 1) / WARPS;
    const int n_my = (int)(w1 - w0);
    const int r_first = (int)(u0 / kc);
    const int r_last = (int)((u1 - 1) / kc);  // valid when len > 0
    const int n_rt = len > 0 ? r_last - r_first + 1 : 0;

    uint8_t* my_slots = smem + (size_t)warp * DEPTH * Plan::SLOT;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFF);
    uint64_t* my_bars = bars + warp * DEPTH;
    uint64_t* xbar = bars + WARPS * DEPTH;
    const uint8_t* my_tiles = v.tiles + (size_t)w0 * TILE;
    float* table = reinterpret_cast<float*>(smem + Plan::table_off(kc));  // [n_rt][WARPS][16]

    // 1. start the weight stream
    if (lane == 0) {
        for (int s = 0; s < DEPTH; ++s) {
            mbar_init(&my_bars[s], 1);
        }
        if (warp == 0) {
            mbar_init(xbar, 1);
        }
        fence_barrier_init();
        for (int s = 0; s < DEPTH && s < n_my; ++s) {
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)s * TILE, TILE, &my_bars[s]);
        }
    }
    {
        uint32_t* z = reinterpret_cast<uint32_t*>(smem + Plan::X_OFF + xpack1_bytes(kc));
        for (int i = threadIdx.x; i < 128; i += WARPS * 32) {
            z[i] = 0u;
        }
        for (int i = threadIdx.x; i < n_rt * WARPS * 16; i += WARPS * 32) {
            table[i] = 0.0f;
        }
    }
    pdl_launch_dependents();
    // 2. everything below may read what the previous kernel in the stream produced
    pdl_wait();

    uint8_t* xbase = smem + Plan::X_OFF;
    const uint32_t xbytes = (uint32_t)xpack1_bytes(kc);
    if (threadIdx.x == 0) {
        mbar_expect_tx(xbar, xbytes);
        bulk_copy_g2s(xbase, xp.xq, xbytes, xbar);
    }
    __syncthreads();  // barriers initialised, zero page and table cleared
    XShared xsrc;
    xsrc.xq = xbase;
    xsrc.xs = reinterpret_cast<const float*>(xbase + xpack1_xs_offset(kc));
    xsrc.xsum = reinterpret_cast<const int2*>(xbase + xpack1_xsum_offset(kc));
    xsrc.zeros = xbase + xbytes;
    xsrc.cur = xbase;
    bool ok = true;
    if (!mbar_wait(xbar, 0)) {
        ok = false;
        if (lane == 0) {
            atomicExch(status, 2);
        }
    }

    // 3. stream this warp's run of tiles
    const int g = lane >> 2;
    const int t = lane & 3;
    float acc[2] = {0.0f, 0.0f};
    int r_cur = n_my > 0 ? (int)(w0 / kc) : 0;
    int c_cur = n_my > 0 ? (int)(w0 % kc) : 0;
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
            compute_chunk_m1<FMT>(my_slots + (size_t)s * Plan::SLOT, xsrc, c_cur, lane, acc);
        }
        __syncwarp();
        if (ok && lane == 0 && i + DEPTH < n_my) {
            fence_proxy_async();  // order this warp's reads of the slot before the refill
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)(i + DEPTH) * TILE, TILE, &my_bars[s]);
        }
        ++c_cur;
        if (c_cur == kc || i + 1 == n_my) {
            // the row tile ends (or this warp's run does): park the sums
            acc[0] += __shfl_xor_sync(0xFFFFFFFFu, acc[0], 1);
            acc[1] += __shfl_xor_sync(0xFFFFFFFFu, acc[1], 1);
            if (t == 0) {
                float* dst = table + ((size_t)(r_cur - r_first) * WARPS + warp) * 16;
                dst[g] = acc[0];
                dst[g + 8] = acc[1];
            }
            acc[0] = acc[1] = 0.0f;
            c_cur = 0;
            ++r_cur;
        }
    }
    __syncthreads();

    // 4. warp 0 finishes the row tiles of this CTA: lanes 0..15 are the 16 rows.  The part
    //    of a row tile that continues in the next CTA is published FIRST, so that no CTA
    //    makes its right neighbour wait for its own left neighbour.
    if (warp == 0 && n_rt > 0) {
        const int i16 = lane & 15;
        int n_own = n_rt;
        if ((long long)(r_last + 1) * kc > u1) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                sum += table[((size_t)(n_rt - 1) * WARPS + w) * 16 + i16];
            }
            if (lane < 16) {
                sk.scratch[j * 16 + i16] = sum;
                __threadfence();
            }
            __syncwarp();
            if (lane == 0) {
                st_release_u32(sk.flags + j, 1u);
            }
            n_own = n_rt - 1;
        }
        for (int rl = 0; rl < n_own; ++rl) {
            const int r = r_first + rl;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                sum += table[((size_t)rl * WARPS + w) * 16 + i16];
            }
            const long long ru0 = (long long)r * kc;
            if (ru0 < u0) {
                // parts of this row tile live in the CTAs to the left; nearest first
                for (long long jp = j - 1; jp >= 0; --jp) {
                    const long long pu1 = U * (jp + 1) / G;
                    if (pu1 <= ru0) {
                        break;
                    }
                    bool ready = false;
                    for (unsigned spin = 0; spin < (1u << 20); ++spin) {
                        if (ld_acquire_u32(sk.flags + jp) != 0u) {
                            ready = true;
                            break;
                        }
                        __nanosleep(32);
                    }
                    if (!ready) {
                        if (lane == 0) {
                            atomicExch(status, 3);
                        }
                        break;
                    }
                    sum += sk.scratch[jp * 16 + i16];
                    __syncwarp();
                    if (lane == 0) {
                        sk.flags[jp] = 0u;  // consumed; the next launch starts from zero
                    }
                }
            }
            const int64_t row = (int64_t)r * 16 + i16;
            if (lane < 16 && row < v.n) {
                y[row] = sum;
            }
        }
    }
}

// Quantize x to 16 bits per (row, 256-chunk) and store it in B-fragment order.
// grid (kc, ncp), 128 threads: warp w handles activation row 4*blockIdx.y + w.
// x ~= xs * (256*hi + lo) with hi and lo both signed bytes.
__global__ void __launch_bounds__(128) pack_x_kernel(const float* __restrict__ x, int m, int64_t k, int kc, int ncp,
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
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t col = (int64_t)c * 256 + 8 * lane + i;
        v[i] = (row < m && col < k) ? x[(int64_t)row * k + col] : 0.0f;
        amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    }
    // |q| <= 32639 = 127*256 + 127 keeps both signed digits inside int8
    const float inv = amax > 0.0f ? 32639.0f / amax : 0.0f;
    int bsum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int qi = __float2int_rn(v[i] * inv);
        qi = max(-32639, min(32639, qi));
        q[warp][8 * lane + i] = (short)qi;
        bsum += qi;
    }
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 1);
    bsum += __shfl_xor_sync(0xFFFFFFFFu, bsum, 2);
    float* xs = reinterpret_cast<float*>(out + (compact ? xpack1_xs_offset(kc) : xpack_xs_offset(kc, ncp)));
    int2* xsum = reinterpret_cast<int2*>(out + (compact ? xpack1_xsum_offset(kc) : xpack_xsum_offset(kc, ncp)));
    if (compact) {
        if (warp == 0) {
            if (lane == 0) {
                xs[c] = amax / 32639.0f;
            }
            if ((lane & 3) == 0) {
                xsum[c * 8 + (lane >> 2)] = make_int2(8 * bsum, 128 * bsum);
            }
        }
    } else {
        if (lane == 0) {
            xs[c * 16 + row] = amax / 32639.0f;
        }
        if ((lane & 3) == 0) {
            xsum[(size_t)(c * 8 + (lane >> 2)) * 16 + row] = make_int2(8 * bsum, 128 * bsum);
        }
    }
    __syncthreads();

    // fragment lane (g,t) of block b: activation row g>>1 of this group, digit g&1
    const int lanes = compact ? 8 : 32;
    uint2* xq = reinterpret_cast<uint2*>(out);
    for (int i = threadIdx.x; i < 8 * lanes; i += 128) {
        const int b = i / lanes;
        const int fl = i % lanes;
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
        if (compact) {
            xq[(size_t)(c * 8 + b) * 8 + fl] = make_uint2(w0, w1);
        } else {
            xq[((size_t)(c * 8 + b) * ncp + j) * 32 + fl] = make_uint2(w0, w1);
        }
    }
}

// Ring depth per format: 28-37 KB of tiles in flight per CTA.
template <int FMT>
struct Tune {
    static constexpr int WARPS = 4;
    static constexpr int DEPTH = FMT == FMT_Q8_0 ? 2 : 3;
};

template <int FMT, int MC, int WARPS, int DEPTH>
cudaError_t launch_gemv_variant(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                                cudaStream_t stream)
{
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
    return cudaLaunchKernelEx(&cfg, kernel, w, xp, y, m, status);
}

// Ring depth of the persistent batch-1 kernel: ~90-105 KB of tiles per SM.
template <int FMT>
struct TuneSK {
    static constexpr int WARPS = 8;
    static constexpr int DEPTH = FMT == FMT_Q8_0 ? 3 : FMT == FMT_Q6_K ? 4 : 5;
};

template <int FMT, int WARPS, int DEPTH>
cudaError_t launch_gemv_streamk(const WeightView& w, const XPackView& xp, float* y, const StreamKArgs& sk, int grid,
                                int* status, cudaStream_t stream)
{
    using Plan = StreamKPlan<FMT, WARPS, DEPTH>;
    auto kernel = gemv_m1_streamk_kernel<FMT, WARPS, DEPTH>;
    const long long U = (long long)w.rt * w.kc;
    const int smem = Plan::total(w.kc, (U + grid - 1) / grid);
    if (smem > 227 * 1024) {
        return cudaErrorInvalidConfiguration;
    }
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
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, w, xp, y, sk, status);
}

template <int FMT, int MC>
cudaError_t launch_gemv_fmt_mc(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                               cudaStream_t stream)
{
    if constexpr (FMT == FMT_Q4_0 && MC == 1) {
        static int tune = -1;
        if (tune < 0) {
            const char* e = getenv("QMM_TUNE");
            tune = e ? atoi(e) : 0;
        }
        switch (tune) {
        case 82: return launch_gemv_variant<FMT, MC, 8, 2>(w, xp, y, m, status, stream);
        case 81: return launch_gemv_variant<FMT, MC, 8, 1>(w, xp, y, m, status, stream);
        case 161: return launch_gemv_variant<FMT, MC, 16, 1>(w, xp, y, m, status, stream);
        case 42: return launch_gemv_variant<FMT, MC, 4, 2>(w, xp, y, m, status, stream);
        case 44: return launch_gemv_variant<FMT, MC, 4, 4>(w, xp, y, m, status, stream);
        case 24: return launch_gemv_variant<FMT, MC, 2, 4>(w, xp, y, m, status, stream);
        default: break;
        }
    }
    return launch_gemv_variant<FMT, MC, Tune<FMT>::WARPS, Tune<FMT>::DEPTH>(w, xp, y, m, status, stream);
}

template <int FMT>
cudaError_t launch_gemv_fmt(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                            cudaStream_t stream)
{
    if (m == 1) {
        return launch_gemv_fmt_mc<FMT, 1>(w, xp, y, m, status, stream);
    }
    if (m <= 4) {
        return launch_gemv_fmt_mc<FMT, 4>(w, xp, y, m, status, stream);
    }
    if (m <= 8) {
        return launch_gemv_fmt_mc<FMT, 8>(w, xp, y, m, status, stream);
    }
    if (m <= 12) {
        return launch_gemv_fmt_mc<FMT, 12>(w, xp, y, m, status, stream);
    }
    return launch_gemv_fmt_mc<FMT, 16>(w, xp, y, m, status, stream);
}

}  // namespace

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
    return cudaLaunchKernelEx(&cfg, pack_x_kernel, x, m, k, kc, ncp, m == 1 ? 1 : 0, out);
}

#ifdef QMM_TRACE
extern "C" int qmm_trace_arm(unsigned long long* buf, unsigned int cap)
{
    unsigned int zero = 0;
    cudaMemcpyToSymbol(g_trace_buf, &buf, sizeof(buf));
    cudaMemcpyToSymbol(g_trace_cap, &cap, sizeof(cap));
    cudaMemcpyToSymbol(g_trace_cursor, &zero, sizeof(zero));
    return (int)cudaDeviceSynchronize();
}
extern "C" unsigned int qmm_trace_count()
{
    unsigned int n = 0;
    cudaMemcpyFromSymbol(&n, g_trace_cursor, sizeof(n));
    return n;
}
#endif

cudaError_t launch_gemv_m1(const WeightView& w, const XPackView& xp, float* y, float* scratch, unsigned int* flags,
                           int grid, int* status, cudaStream_t stream)
{
    StreamKArgs sk;
    sk.scratch = scratch;
    sk.flags = flags;
    int variant = 0;
    if (const char* e = getenv("QMM_TUNE")) {
        variant = atoi(e);
    }
    switch (w.fmt) {
    case FMT_Q4_0:
        if (variant == 322) return launch_gemv_streamk<FMT_Q4_0, 32, 2>(w, xp, y, sk, grid, status, stream);
        if (variant == 323) return launch_gemv_streamk<FMT_Q4_0, 32, 3>(w, xp, y, sk, grid, status, stream);
        if (variant == 242) return launch_gemv_streamk<FMT_Q4_0, 24, 2>(w, xp, y, sk, grid, status, stream);
        if (variant == 84) return launch_gemv_streamk<FMT_Q4_0, 8, 4>(w, xp, y, sk, grid, status, stream);
        if (variant == 86) return launch_gemv_streamk<FMT_Q4_0, 8, 6>(w, xp, y, sk, grid, status, stream);
        if (variant == 163) return launch_gemv_streamk<FMT_Q4_0, 16, 3>(w, xp, y, sk, grid, status, stream);
        if (variant == 162) return launch_gemv_streamk<FMT_Q4_0, 16, 2>(w, xp, y, sk, grid, status, stream);
        if (variant == 48) return launch_gemv_streamk<FMT_Q4_0, 4, 8>(w, xp, y, sk, grid, status, stream);
        return launch_gemv_streamk<FMT_Q4_0, TuneSK<FMT_Q4_0>::WARPS, TuneSK<FMT_Q4_0>::DEPTH>(w, xp, y, sk, grid, status,
                                                                                                stream);
    case FMT_Q8_0:
        return launch_gemv_streamk<FMT_Q8_0, TuneSK<FMT_Q8_0>::WARPS, TuneSK<FMT_Q8_0>::DEPTH>(w, xp, y, sk, grid, status,
                                                                                                stream);
    case FMT_Q4_K:
        return launch_gemv_streamk<FMT_Q4_K, TuneSK<FMT_Q4_K>::WARPS, TuneSK<FMT_Q4_K>::DEPTH>(w, xp, y, sk, grid, status,
                                                                                                stream);
    case FMT_Q6_K:
        return launch_gemv_streamk<FMT_Q6_K, TuneSK<FMT_Q6_K>::WARPS, TuneSK<FMT_Q6_K>::DEPTH>(w, xp, y, sk, grid, status,
                                                                                                stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemv(const WeightView& w, const XPackView& xp, float* y, int m, int* status, cudaStream_t stream)
{
    switch (w.fmt) {
    case FMT_Q4_0: return launch_gemv_fmt<FMT_Q4_0>(w, xp, y, m, status, stream);
    case FMT_Q8_0: return launch_gemv_fmt<FMT_Q8_0>(w, xp, y, m, status, stream);
    case FMT_Q4_K: return launch_gemv_fmt<FMT_Q4_K>(w, xp, y, m, status, stream);
    case FMT_Q6_K: return launch_gemv_fmt<FMT_Q6_K>(w, xp, y, m, status, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace qmm

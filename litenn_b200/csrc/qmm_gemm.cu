// Prefill GEMM on the 5th-generation tensor cores (sm_100a): Y[M,N] = X[M,K] · Wᵀ with bf16
// activations, block-quantized weights dequantized on the fly, fp32 accumulation in TMEM.
//
// One CTA owns up to 256 activation rows (two 128-row UMMA tiles) and a contiguous group
// of up to 16 row tiles of the weight (n <= 256 output features); its accumulators fill
// 2 x n <= 512 TMEM columns, so every weight tile is dequantized once per CTA and reused
// for all its activation rows.  Per 64-wide K step:
//   warp 0          TMA: two 128x64 bf16 boxes of X -> shared memory (128-byte swizzle)
//   warps 2..17     read the packed weight tiles (qmm_common.cuh) from global memory,
//                   rebuild the exact fp32 values ggml's to_float gives, round them to bf16
//                   and store them as the K-major, 128-byte-swizzled B tile
//   warp 1, lane 0  tcgen05.mma (kind::f16, bf16 x bf16 -> fp32, M=128, N=n, K=16) x 4 x 2,
//                   then tcgen05.commit to hand the stage back
// A 3-stage mbarrier ring decouples the three roles.  At the end warps 2..5 read the
// accumulators with tcgen05.ld and write Y.  Every wait has an iteration limit; a CTA
// that gives up sets the status word, still frees its TMEM and returns.
#include <cuda.h>

#include <cstdlib>
#include <cuda_bf16.h>

#include "qmm_kernels.h"

namespace qmm {

namespace {

constexpr int GEMM_STAGES = 3;
constexpr int GEMM_BK = 64;                    // K per stage: 128 bytes of bf16 = one swizzle row
constexpr int GEMM_A_TILE_BYTES = 128 * 128;   // 128 rows x 64 bf16
constexpr int GEMM_A_STAGE_BYTES = 2 * GEMM_A_TILE_BYTES;
constexpr int GEMM_B_STAGE_BYTES = 256 * 128;  // up to 256 weight rows x 64 bf16
constexpr int GEMM_STAGE_BYTES = GEMM_A_STAGE_BYTES + GEMM_B_STAGE_BYTES;
constexpr int GEMM_DEQ_WARPS = 16;
constexpr int GEMM_THREADS = (2 + GEMM_DEQ_WARPS) * 32;
constexpr int GEMM_SMEM_BYTES = GEMM_STAGES * GEMM_STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr uint32_t GEMM_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t g_smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void g_mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(g_smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void g_mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(g_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void g_mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(g_smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool g_mbar_wait(uint64_t* bar, uint32_t parity)
{
    const uint32_t addr = g_smem_u32(bar);
    for (uint32_t spin = 0; spin < GEMM_SPIN_LIMIT; ++spin) {
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

// Same with a non-suspending probe: used by single elected threads that sit on the critical
// path of the stage hand-over (a suspended try_wait wakes up late).
__device__ __forceinline__ bool g_mbar_poll(uint64_t* bar, uint32_t parity)
{
    const uint32_t addr = g_smem_u32(bar);
    for (uint32_t spin = 0; spin < (GEMM_SPIN_LIMIT << 4); ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
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

// 2-D tiled TMA load (no multicast): box {64 k, 128 rows} at element coordinates (k0, row0).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int k0, int row0, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            g_smem_u32(dst)),
        "l"(map), "r"(k0), "r"(row0), "r"(g_smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                          // 128-byte swizzle
    return d;
}

// Instruction descriptor: D fp32, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(g_smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Byte offset of element (row, k) of a K-major tile with 128-byte rows and 128-byte swizzle:
// the 16-byte chunk index is XORed with the row index modulo 8.
__device__ __forceinline__ uint32_t swz128(int row, int k)
{
    const uint32_t chunk = (uint32_t)(k >> 3) ^ (uint32_t)(row & 7);
    return (uint32_t)row * 128u + chunk * 16u + (uint32_t)(k & 7) * 2u;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Store four consecutive k values (k0 multiple of 4) of one row: 8 bytes inside one 16-byte chunk.
__device__ __forceinline__ void store_b4(uint8_t* btile, int row, int k0, float v0, float v1, float v2, float v3)
{
    *reinterpret_cast<uint2*>(btile + swz128(row, k0)) = make_uint2(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3));
}

// ---- dequantization of one 16-row x 64-column piece into the B tile --------------------------

// What one lane keeps of a (row tile, 64-wide K step): quant words and scale words.
struct PackedRegs {
    uint32_t w[8];
    uint32_t s[8];
};

__device__ __forceinline__ uint32_t ldg_u32(const uint8_t* p)
{
    return __ldg(reinterpret_cast<const uint32_t*>(p));
}

// `tile` points at the packed 16x256 tile, q (0..3) selects the 64-wide quarter of it.
template <int FMT>
__device__ __forceinline__ void load_packed(PackedRegs& r, const uint8_t* tile, int q, int lane)
{
    const int g = lane >> 2;
    const uint8_t* p1 = tile + tile_p1_offset(FMT);
    const uint8_t* p2 = tile + tile_p2_offset(FMT);
    if constexpr (FMT == FMT_Q4_0 || FMT == FMT_Q4_K) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(tile) + q * 32 + lane);
        r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
        if constexpr (FMT == FMT_Q4_0) {
            r.s[0] = ldg_u32(p1 + g * 16 + 4 * q);        // fp16 d of blocks 2q, 2q+1, row g
            r.s[1] = ldg_u32(p1 + (g + 8) * 16 + 4 * q);  // row g+8
        } else {
#pragma unroll
            for (int rs = 0; rs < 2; ++rs) {
                const uint8_t* sp = p1 + (g + 8 * rs) * 12;
                r.s[4 * rs + 0] = ldg_u32(sp);
                r.s[4 * rs + 1] = ldg_u32(sp + 4);
                r.s[4 * rs + 2] = ldg_u32(sp + 8);
                r.s[4 * rs + 3] = ldg_u32(p2 + (g + 8 * rs) * 4);  // (d, dmin)
            }
        }
    } else if constexpr (FMT == FMT_Q8_0) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(tile) + (2 * q) * 32 + lane);
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(tile) + (2 * q + 1) * 32 + lane);
        r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w;
        r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
        r.s[0] = ldg_u32(p1 + g * 16 + 4 * q);
        r.s[1] = ldg_u32(p1 + (g + 8) * 16 + 4 * q);
    } else {  // Q6_K: quarter q = sub-blocks 4q..4q+3; words (q*2+rsel)*3 + {0,1,2} of this lane
#pragma unroll
        for (int rs = 0; rs < 2; ++rs) {
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int W = (q * 2 + rs) * 3 + j;
                r.w[3 * rs + j] = ldg_u32(tile + (((W >> 2) * 32 + lane) * 4 + (W & 3)) * 4);
            }
            r.s[rs] = ldg_u32(p1 + (g + 8 * rs) * 16 + 4 * q);  // int8 scales of sub-blocks 4q..4q+3
            r.s[2 + rs] = __ldg(reinterpret_cast<const unsigned short*>(p2 + (g + 8 * rs) * 2));
        }
    }
}

__device__ __forceinline__ float h2f_bits(uint32_t bits16)
{
    return __half2float(__ushort_as_half((unsigned short)(bits16 & 0xFFFFu)));
}

// Writes rows (16*rl + g) and (16*rl + g + 8), 64 columns, of the B tile.  The fp32 value of
// every weight is computed with the same roundings as ggml's to_float, then rounded to bf16.
template <int FMT>
__device__ __forceinline__ void dequant_to_btile(const PackedRegs& r, uint8_t* btile, int rl, int q, int lane)
{
    const int g = lane >> 2;
    const int t = lane & 3;
    const int row0 = 16 * rl + g;
    if constexpr (FMT == FMT_Q4_0) {
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            // word wi: block 2q + (wi>>1), weights 16*(wi&1) + 4t.. -> column 32*(wi>>1) + 16*(wi&1) + 4t
            const int k0 = 32 * (wi >> 1) + 16 * (wi & 1) + 4 * t;
            const uint32_t w = r.w[wi];
#pragma unroll
            for (int rs = 0; rs < 2; ++rs) {
                const float d = h2f_bits(r.s[rs] >> (16 * (wi >> 1)));
                float v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = (int)((w >> (8 * i + 4 * rs)) & 15u);
                    v[i] = __fmul_rn((float)(n - 8), d);
                }
                store_b4(btile, row0 + 8 * rs, k0, v[0], v[1], v[2], v[3]);
            }
        }
    } else if constexpr (FMT == FMT_Q8_0) {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // word j of block b: row g + 8*(j&1), bytes 16*(j>>1) + 4t..
                const int rs = j & 1;
                const int k0 = 32 * b + 16 * (j >> 1) + 4 * t;
                const uint32_t w = r.w[4 * b + j];
                const float d = h2f_bits(r.s[rs] >> (16 * b));
                float v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[i] = __fmul_rn((float)(int)(signed char)((w >> (8 * i)) & 0xFFu), d);
                }
                store_b4(btile, row0 + 8 * rs, k0, v[0], v[1], v[2], v[3]);
            }
        }
    } else if constexpr (FMT == FMT_Q4_K) {
        // this quarter holds sub-blocks 2q and 2q+1
#pragma unroll
        for (int rs = 0; rs < 2; ++rs) {
            const uint32_t w0 = r.s[4 * rs + 0], w1 = r.s[4 * rs + 1], w2 = r.s[4 * rs + 2];
            const uint32_t scw = q < 2 ? (w0 & 0x3F3F3F3Fu) : ((w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u));
            const uint32_t mnw = q < 2 ? (w1 & 0x3F3F3F3Fu) : (((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u));
            const float d = h2f_bits(r.s[4 * rs + 3]);
            const float dmin = h2f_bits(r.s[4 * rs + 3] >> 16);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int byte = (2 * q + h) & 3;
                const float d1 = __fmul_rn(d, (float)((scw >> (8 * byte)) & 0xFFu));
                const float m1 = __fmul_rn(dmin, (float)((mnw >> (8 * byte)) & 0xFFu));
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t w = r.w[2 * h + half];
                    const int k0 = 32 * h + 16 * half + 4 * t;
                    float v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int n = (int)((w >> (8 * i + 4 * rs)) & 15u);
                        v[i] = __fsub_rn(__fmul_rn(d1, (float)n), m1);
                    }
                    store_b4(btile, row0 + 8 * rs, k0, v[0], v[1], v[2], v[3]);
                }
            }
        }
    } else {  // Q6_K
#pragma unroll
        for (int rs = 0; rs < 2; ++rs) {
            const uint32_t X = r.w[3 * rs + 0], Y = r.w[3 * rs + 1], Z = r.w[3 * rs + 2];
            const float d = h2f_bits(r.s[2 + rs]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float ds = __fmul_rn(d, (float)(int)(signed char)((r.s[rs] >> (8 * j)) & 0xFFu));
                float v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t u;
                    if (j < 3) {
                        const uint32_t word = j == 0 ? X : (j == 1 ? Y : Z);
                        u = ((word >> (8 * i)) & 0xFFu) >> 2;
                    } else {
                        u = (((X >> (8 * i)) & 3u) << 4) | (((Y >> (8 * i)) & 3u) << 2) | ((Z >> (8 * i)) & 3u);
                    }
                    const int qv = (int)(u ^ 32u) - 32;
                    v[i] = __fmul_rn(ds, (float)qv);
                }
                store_b4(btile, row0 + 8 * rs, 16 * j + 4 * t, v[0], v[1], v[2], v[3]);
            }
        }
    }
}

// ---- the kernel -----------------------------------------------------------------------------

struct GemmArgs {
    WeightView w;
    void* y;            // [M, N] row-major, fp32 or bf16
    int64_t m;
    int out_bf16;
    int groups_per_tg;  // CTAs that share one group of 256 activation rows
    int* status;
};


template <int FMT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap xmap, const GemmArgs args)
{
    extern __shared__ uint8_t gemm_smem_raw[];
    // the swizzle pattern is defined on absolute shared-memory addresses: 1024-byte alignment
    uint8_t* smem = gemm_smem_raw + ((1024u - (g_smem_u32(gemm_smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GEMM_STAGES * GEMM_STAGE_BYTES);
    uint64_t* full_a = bars;                    // [STAGES]  TMA bytes landed
    uint64_t* full_b = bars + GEMM_STAGES;      // [STAGES]  dequant warps done
    uint64_t* empty = bars + 2 * GEMM_STAGES;   // [STAGES]  MMAs that read the stage have completed
    uint64_t* accum = bars + 3 * GEMM_STAGES;   // all MMAs completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * GEMM_STAGES + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const WeightView& v = args.w;
    const int tg = blockIdx.x / args.groups_per_tg;
    const int gi = blockIdx.x % args.groups_per_tg;
    const int rt0 = (int)((long long)v.rt * gi / args.groups_per_tg);
    const int rt1 = (int)((long long)v.rt * (gi + 1) / args.groups_per_tg);
    const int R = rt1 - rt0;        // row tiles of this CTA, 1..16
    const int n = R * 16;           // UMMA N
    const int64_t row_base = (int64_t)tg * 256;
    const int ntt = (args.m - row_base) > 128 ? 2 : 1;
    const int n_stages = (int)((v.k + GEMM_BK - 1) / GEMM_BK);
    // CTAs that share activation rows start at different K offsets (the sum does not care
    // about the order), so they do not all ask L2 for the same lines at the same moment.
    const int k_rot = (int)((long long)n_stages * gi / args.groups_per_tg);

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; ++s) {
            g_mbar_init(&full_a[s], 1);
            g_mbar_init(&full_b[s], GEMM_DEQ_WARPS);
            g_mbar_init(&empty[s], 1);
        }
        g_mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // 512 columns: two accumulators of up to 256 columns each
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(g_smem_u32(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer: activations ----
        if (lane == 0) {
            for (int s = 0; s < n_stages; ++s) {
                const int slot = s % GEMM_STAGES;
                if (s >= GEMM_STAGES && !g_mbar_poll(&empty[slot], (uint32_t)(s / GEMM_STAGES - 1) & 1u)) {
                    atomicExch(args.status, 11);
                    break;
                }
                uint8_t* a = smem + (size_t)slot * GEMM_STAGE_BYTES;
                g_mbar_expect_tx(&full_a[slot], (uint32_t)(ntt * GEMM_A_TILE_BYTES));
                const int ks = (s + k_rot) % n_stages;
                tma_load_2d(a, &xmap, ks * GEMM_BK, (int)row_base, &full_a[slot]);
                if (ntt == 2) {
                    tma_load_2d(a + GEMM_A_TILE_BYTES, &xmap, ks * GEMM_BK, (int)row_base + 128, &full_a[slot]);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(n);
            bool ok = true;
            for (int s = 0; s < n_stages && ok; ++s) {
                const int slot = s % GEMM_STAGES;
                const uint32_t parity = (uint32_t)(s / GEMM_STAGES) & 1u;
                if (!g_mbar_poll(&full_a[slot], parity) || !g_mbar_poll(&full_b[slot], parity)) {
                    atomicExch(args.status, 12);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = g_smem_u32(smem + (size_t)slot * GEMM_STAGE_BYTES);
                const uint32_t b_addr = a_addr + GEMM_A_STAGE_BYTES;
#pragma unroll
                for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
                    const uint64_t db = umma_smem_desc(b_addr + kk * 32);
                    for (int tt = 0; tt < ntt; ++tt) {
                        const uint64_t da = umma_smem_desc(a_addr + tt * GEMM_A_TILE_BYTES + kk * 32);
                        umma_bf16(tmem_base + (uint32_t)tt * 256u, da, db, idesc, (s > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&empty[slot]);  // arrives when the MMAs above have read their operands
            }
            if (ok) {
                umma_commit(accum);
            }
        }
    } else {
        // ---- dequant producers: weights -> bf16 B tile ----
        const int dw = warp - 2;  // 0..15: row tile dw of this CTA
        const bool has0 = dw < R;
        // Three register sets rotate: a set is refilled with the packed words of the K step
        // three ahead as soon as it has been converted, so global-memory latency is covered
        // by three steps of work.
        PackedRegs pa0 = {}, pb0 = {}, pc0 = {};
        const size_t tile_stride = tile_bytes(FMT);
        const uint8_t* t0 = v.tiles + ((size_t)(rt0 + dw) * v.kc) * tile_stride;
        auto fetch = [&](int s, PackedRegs& p0) {
            if (s < n_stages && has0) {
                const int ks = (s + k_rot) % n_stages;
                load_packed<FMT>(p0, t0 + (size_t)(ks >> 2) * tile_stride, ks & 3, lane);
            }
        };
        bool ok = true;
        auto step = [&](int s, PackedRegs& p0) {
            if (!ok || s >= n_stages) {
                return;
            }
            const int slot = s % GEMM_STAGES;
            const int ks = (s + k_rot) % n_stages;
            if ((ks & 3) == 0) {
                // pull the packed tiles two K chunks ahead into L2, one 128-byte line per lane
                const int cpre = (ks >> 2) + 2;
                if (cpre < v.kc && lane * 128 < (int)tile_stride) {
                    if (has0) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(t0 + (size_t)cpre * tile_stride + lane * 128));
                    }
                }
            }
            if (s >= GEMM_STAGES) {
                // lane 0 probes, the others wait for it at the warp barrier
                bool landed = true;
                if (lane == 0) {
                    landed = g_mbar_poll(&empty[slot], (uint32_t)(s / GEMM_STAGES - 1) & 1u);
                }
                landed = __shfl_sync(0xFFFFFFFFu, landed, 0);
                if (!landed) {
                    if (lane == 0) {
                        atomicExch(args.status, 13);
                    }
                    ok = false;
                    return;
                }
            }
            uint8_t* btile = smem + (size_t)slot * GEMM_STAGE_BYTES + GEMM_A_STAGE_BYTES;
            if (has0) {
                dequant_to_btile<FMT>(p0, btile, dw, ks & 3, lane);
            }
            // make the generic-proxy stores visible to the tensor core (async proxy), then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                g_mbar_arrive(&full_b[slot]);
            }
            fetch(s + 3, p0);
        };
        fetch(0, pa0);
        fetch(1, pb0);
        fetch(2, pc0);
        for (int s = 0; s < n_stages; s += 3) {
            step(s, pa0);
            step(s + 1, pb0);
            step(s + 2, pc0);
        }

        // ---- epilogue: warps 2..5 own TMEM lanes 32*(warp%4).. ----
        if (warp < 6) {
            if (!g_mbar_wait(accum, 0)) {
                if (lane == 0) {
                    atomicExch(args.status, 14);
                }
            } else {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int quad = warp & 3;
                for (int tt = 0; tt < ntt; ++tt) {
                    const int64_t row = row_base + 128 * tt + 32 * quad + lane;
                    for (int c0 = 0; c0 < n; c0 += 32) {
                        uint32_t acc[32];
                        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(32 * quad) << 16) + (uint32_t)(tt * 256 + c0), acc);
                        if (row < args.m) {
                            const int64_t col0 = (int64_t)rt0 * 16 + c0;
                            // 8 columns at a time: 16-byte (bf16) or 2 x 16-byte (fp32) stores when
                            // the row pitch keeps them aligned, scalar stores at ragged edges
                            if (args.out_bf16) {
                                __nv_bfloat16* yo = static_cast<__nv_bfloat16*>(args.y) + row * v.n + col0;
                                const bool vec = (v.n & 7) == 0;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    if (vec && c0 + 8 * j + 8 <= n && col0 + 8 * j + 8 <= v.n) {
                                        uint4 o;
                                        o.x = pack_bf16x2(__uint_as_float(acc[8 * j + 0]), __uint_as_float(acc[8 * j + 1]));
                                        o.y = pack_bf16x2(__uint_as_float(acc[8 * j + 2]), __uint_as_float(acc[8 * j + 3]));
                                        o.z = pack_bf16x2(__uint_as_float(acc[8 * j + 4]), __uint_as_float(acc[8 * j + 5]));
                                        o.w = pack_bf16x2(__uint_as_float(acc[8 * j + 6]), __uint_as_float(acc[8 * j + 7]));
                                        *reinterpret_cast<uint4*>(yo + 8 * j) = o;
                                    } else {
#pragma unroll
                                        for (int i = 8 * j; i < 8 * j + 8; ++i) {
                                            if (col0 + i < v.n && c0 + i < n) {
                                                yo[i] = __float2bfloat16_rn(__uint_as_float(acc[i]));
                                            }
                                        }
                                    }
                                }
                            } else {
                                float* yo = static_cast<float*>(args.y) + row * v.n + col0;
                                const bool vec = (v.n & 3) == 0;
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (vec && c0 + 4 * j + 4 <= n && col0 + 4 * j + 4 <= v.n) {
                                        *reinterpret_cast<uint4*>(yo + 4 * j) =
                                            make_uint4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                                    } else {
#pragma unroll
                                        for (int i = 4 * j; i < 4 * j + 4; ++i) {
                                            if (col0 + i < v.n && c0 + i < n) {
                                                yo[i] = __uint_as_float(acc[i]);
                                            }
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}


// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

template <int FMT>
cudaError_t launch_gemm_fmt(const CUtensorMap& xmap, const GemmArgs& args, int grid, cudaStream_t stream)
{
    auto kernel = gemm_tcgen05_kernel<FMT>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
        if (e != cudaSuccess) {
            return e;
        }
        if (dev >= 0 && dev < 64) {
            configured[dev] = true;
        }
    }
    kernel<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, stream>>>(xmap, args);
    return cudaGetLastError();
}

}  // namespace


cudaError_t launch_gemm_bf16(const WeightView& w, const void* x_bf16, void* y, int64_t m, int out_bf16, int sm_count,
                             int* status, cudaStream_t stream, const char** why)
{
    *why = nullptr;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) {
        *why = "cuTensorMapEncodeTiled is not available from the driver";
        return cudaErrorNotSupported;
    }
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0 || (w.k % 8) != 0) {
        *why = "activations must be 16-byte aligned with a row length that is a multiple of 8";
        return cudaErrorInvalidValue;
    }
    CUtensorMap xmap;
    const cuuint64_t dims[2] = {(cuuint64_t)w.k, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)w.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)GEMM_BK, 128u};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult cr = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), dims, strides, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        *why = "cuTensorMapEncodeTiled rejected the activation tensor";
        return cudaErrorInvalidValue;
    }
    // Work split: groups of 256 activation rows x groups of <= 16 weight row tiles, sized so that
    // one wave of CTAs covers the SMs as evenly as whole row tiles allow.
    const int tgs = (int)((m + 255) / 256);
    int per_tg = sm_count / tgs;
    const int min_per_tg = (w.rt + 15) / 16;
    if (per_tg < min_per_tg) {
        per_tg = min_per_tg;
    }
    if (per_tg > w.rt) {
        per_tg = w.rt;
    }
    GemmArgs args;
    args.w = w;
    args.y = y;
    args.m = m;
    args.out_bf16 = out_bf16;
    args.groups_per_tg = per_tg;
    args.status = status;
    const int grid = tgs * per_tg;
    switch (w.fmt) {
    case FMT_Q4_0: return launch_gemm_fmt<FMT_Q4_0>(xmap, args, grid, stream);
    case FMT_Q8_0: return launch_gemm_fmt<FMT_Q8_0>(xmap, args, grid, stream);
    case FMT_Q4_K: return launch_gemm_fmt<FMT_Q4_K>(xmap, args, grid, stream);
    case FMT_Q6_K: return launch_gemm_fmt<FMT_Q6_K>(xmap, args, grid, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace qmm

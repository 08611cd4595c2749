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
#include "qmm_gemv_device.cuh"
#include "qmm_kernels.h"

namespace qmm {

namespace {

// ---- the kernel -----------------------------------------------------------------------------

// Shared memory of one CTA, carved from the dynamic allocation:
//   slots  WARPS*DEPTH x (tile [+ batches 2..16: that chunk's packed activations]) | mbarriers
//   (+1 for the activations) | (batch 1) all packed activations + 512 zero bytes | cross-warp reduction
template <int FMT, int MC, int WARPS, int DEPTH>
struct SmemPlan {
    static constexpr int XCHUNK = MC == 1 ? 0 : XSlot<Cols<MC>::NCP>::BYTES;
    static constexpr int SLOT = tile_bytes(FMT) + XCHUNK;
    static constexpr int SLOTS_BYTES = WARPS * DEPTH * SLOT;
    static constexpr int BAR_OFF = SLOTS_BYTES;
    static constexpr int BAR_BYTES = (((WARPS * DEPTH + 1) * 8 + 15) / 16) * 16;
    static constexpr int X_OFF = BAR_OFF + BAR_BYTES;
    __host__ __device__ static int x_bytes(int kc, int mc) { return mc == 1 ? (int)xpack1_bytes(kc) + 512 : 0; }
    __host__ __device__ static int red_off(int kc, int mc) { return X_OFF + x_bytes(kc, mc); }
    __host__ __device__ static int total(int kc, int mc) { return red_off(kc, mc) + WARPS * 16 * mc * 4; }
};

// Batches 2..16: the packed activations of chunk c (three pieces of the packed buffer) into the
// slot behind the tile; the second of the slot phase's two arrivals carries their byte count.
template <int MC>
__device__ __forceinline__ void copy_x_chunk(uint8_t* dst, const XPackView& xp, int c, uint64_t* bar)
{
    using XS = XSlot<Cols<MC>::NCP>;
    mbar_expect_tx(bar, XS::BYTES);
    bulk_copy_g2s(dst, xp.xq + (size_t)c * XS::XQ_BYTES, XS::XQ_BYTES, bar);
    bulk_copy_g2s(dst + XS::XQ_BYTES, reinterpret_cast<const uint8_t*>(xp.xs) + (size_t)c * XS::XS_BYTES, XS::XS_BYTES,
                  bar);
    bulk_copy_g2s(dst + XS::XQ_BYTES + XS::XS_BYTES, reinterpret_cast<const uint8_t*>(xp.xsum) + (size_t)c * XS::XSUM_BYTES,
                  XS::XSUM_BYTES, bar);
}

template <int FMT, int MC, int WARPS, int DEPTH>
__global__ void __launch_bounds__(WARPS * 32)
    gemv_kernel(WeightView v, XPackView xp, float* __restrict__ y, int m, int* __restrict__ status, PeerScatter ps)
{
    using Plan = SmemPlan<FMT, MC, WARPS, DEPTH>;
    constexpr int NOUT = Cols<MC>::NOUT;
    constexpr uint32_t TILE = tile_bytes(FMT);
    extern __shared__ __align__(128) uint8_t smem[];

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
    // (batches 2..16: a slot's phase takes two arrivals, one with the tile's bytes, issued here, and
    // one with the chunk's activation bytes, which can only be issued after the dependency wait)
    if (lane == 0) {
        for (int s = 0; s < DEPTH; ++s) {
            mbar_init(&my_bars[s], MC == 1 ? 1 : 2);
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
    // the exchange number depends only on the token position, which earlier tokens set
    unsigned int epoch = 0;
    if constexpr (MC == 1) {
        if (ps.n_peers > 0) {
            epoch = (unsigned int)(*ps.pos * ps.sites + ps.site + 1);
        }
    }
    // 2. everything below may read what the previous kernel in the stream produced
    pdl_wait();

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
        xsrc.base = nullptr;
        if (lane == 0) {
            for (int s = 0; s < DEPTH && s < n_my; ++s) {
                copy_x_chunk<MC>(my_slots + (size_t)s * Plan::SLOT + TILE, xp, warp + s * WARPS, &my_bars[s]);
            }
        }
    }

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
        if (ok) {
            if constexpr (MC == 1) {
                compute_chunk_m1<FMT>(my_slots + (size_t)s * Plan::SLOT, xsrc, warp + i * WARPS, lane, acc);
            } else {
                xsrc.attach(my_slots + (size_t)s * Plan::SLOT + TILE);
                compute_chunk<FMT, MC>(my_slots + (size_t)s * Plan::SLOT, xsrc, warp + i * WARPS, lane, acc);
            }
        }
        __syncwarp();
        if (ok && lane == 0 && i + DEPTH < n_my) {
            fence_proxy_async();  // order this warp's reads of the slot before the refill
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)(warp + (i + DEPTH) * WARPS) * TILE,
                          TILE, &my_bars[s]);
            if constexpr (MC > 1) {
                copy_x_chunk<MC>(my_slots + (size_t)s * Plan::SLOT + TILE, xp, warp + (i + DEPTH) * WARPS, &my_bars[s]);
            }
        }
    }

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
            if constexpr (MC == 1) {
                if (ps.n_peers > 0) {
#pragma unroll
                    for (int p = 0; p < QMM_MAX_PEERS; ++p) {  // over NVLink into the peer's receive buffer
                        if (p < ps.n_peers) {
                            asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(ps.dst[p] + row),
                                         "r"(__float_as_uint(sum)), "r"(epoch)
                                         : "memory");
                        }
                    }
                }
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
                                const PeerScatter& ps, cudaStream_t stream)
{
    using Plan = SmemPlan<FMT, MC, WARPS, DEPTH>;
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
    return cudaLaunchKernelEx(&cfg, kernel, w, xp, y, m, status, ps);
}

template <int FMT, int MC>
cudaError_t launch_gemv_fmt_mc(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                               const PeerScatter& ps, cudaStream_t stream)
{
    if constexpr (MC == 1) {
        // Long rows (K > 4096): with four warps a warp would walk 6-28 tiles one after the other, and
        // in a chain of dependent matvecs that walk starts only when the activations arrive.  More
        // warps per row tile shorten it, as long as two CTAs still fit on an SM.
        constexpr int LIMIT = 113 * 1024;
        // K of 2304..4096: eight warps with one slot each (the whole row tile is in flight from the
        // first instruction, 18 KB per CTA, seven CTAs per SM) measured faster than four warps with
        // three slots for every format but Q8_0, whose larger tiles would drop to four CTAs per SM.
        if (w.kc > 8 && w.kc <= 16 && FMT != FMT_Q8_0) {
            return launch_gemv_variant<FMT, 1, 8, 1>(w, xp, y, m, status, ps, stream);
        }
        if (w.kc > 32 && SmemPlan<FMT, 1, 16, 2>::total(w.kc, 1) <= LIMIT) {
            return launch_gemv_variant<FMT, 1, 16, 2>(w, xp, y, m, status, ps, stream);
        }
        if (w.kc > 16 && SmemPlan<FMT, 1, 8, 3>::total(w.kc, 1) <= LIMIT) {
            return launch_gemv_variant<FMT, 1, 8, 3>(w, xp, y, m, status, ps, stream);
        }
    }
    // batches 2..16 carry 3-9 KB of activations per slot: a shallower ring keeps 2-3 CTAs per SM
    constexpr int DEPTH = MC == 1 ? Tune<FMT>::DEPTH : (MC == 4 && FMT != FMT_Q8_0 ? 3 : 2);
    return launch_gemv_variant<FMT, MC, Tune<FMT>::WARPS, DEPTH>(w, xp, y, m, status, ps, stream);
}

template <int FMT>
cudaError_t launch_gemv_fmt(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                            const PeerScatter& ps, cudaStream_t stream)
{
    if (m == 1) {
        return launch_gemv_fmt_mc<FMT, 1>(w, xp, y, m, status, ps, stream);
    }
    if (m <= 4) {
        return launch_gemv_fmt_mc<FMT, 4>(w, xp, y, m, status, ps, stream);
    }
    if (m <= 8) {
        return launch_gemv_fmt_mc<FMT, 8>(w, xp, y, m, status, ps, stream);
    }
    if (m <= 12) {
        return launch_gemv_fmt_mc<FMT, 12>(w, xp, y, m, status, ps, stream);
    }
    return launch_gemv_fmt_mc<FMT, 16>(w, xp, y, m, status, ps, stream);
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


cudaError_t launch_gemv_scatter(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                                const PeerScatter& ps, cudaStream_t stream)
{
    if (ps.n_peers > 0 && m != 1) {
        return cudaErrorInvalidValue;
    }
    switch (w.fmt) {
    case FMT_Q4_0: return launch_gemv_fmt<FMT_Q4_0>(w, xp, y, m, status, ps, stream);
    case FMT_Q8_0: return launch_gemv_fmt<FMT_Q8_0>(w, xp, y, m, status, ps, stream);
    case FMT_Q4_K: return launch_gemv_fmt<FMT_Q4_K>(w, xp, y, m, status, ps, stream);
    case FMT_Q6_K: return launch_gemv_fmt<FMT_Q6_K>(w, xp, y, m, status, ps, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemv(const WeightView& w, const XPackView& xp, float* y, int m, int* status, cudaStream_t stream)
{
    PeerScatter none = {};
    return launch_gemv_scatter(w, xp, y, m, status, none, stream);
}

}  // namespace qmm

// Dequant-fused GEMV / skinny GEMM for decode (1..16 activation rows) on sm_100a: the kernel
// template and its per-format launcher.  Each block format instantiates it in a translation
// unit of its own (qmm_gemv_q4_0.cu, ...), so the formats compile in parallel.
//
// The weights never become floats in memory.  One CTA owns one 16-row tile of the
// output; its warps take the 256-column K chunks of that row tile round-robin.
// Every chunk is one contiguous packed tile (qmm_common.cuh) that a single TMA bulk
// copy (cp.async.bulk, completion counted on an mbarrier) lands in a shared-memory
// slot.  Each warp owns DEPTH slots and refills a slot itself as soon as it has
// consumed it, so the copies of a whole CTA are in flight from the first instruction
// on and HBM latency is paid once, not per chunk.  From shared memory the quants become
// int8 MMA A-fragments with two or three logic ops per word and are multiplied on the
// integer tensor-core path (mma.sync m16n8k32 / m16n8k16, s32 accumulate) with the
// activations, quantized to 16 bits per 32-wide block and split into a signed high and a
// signed low byte.  The int32 block sums are exact; they are folded into fp32 accumulators
// with the block's fp16 weight scale and the block's activation scale, so the accumulation
// across blocks is fp32 as in the reference loop (src/LiteNN/Device.h:645-658).  The only
// approximation is the 16-bit activation quantization (relative error <= 2^-16 of the
// block maximum).
//
// Kernels are launched with programmatic dependent launch: the weight copies are issued
// before griddepcontrol.wait, so in a chain of dependent matvecs the next kernel's weights
// stream while the previous kernel drains.  Batch 1 brings all packed activations into
// shared memory with one more bulk copy; batches 2..16 bring each chunk's record into the
// ring slot behind the tile.
//
// Fused forms (batch 1, GemvFuse in qmm_common.cuh) let a chain of matvecs run without glue
// kernels between them: a matvec can pack its own fp32 input, apply the scalar 1/rms of an
// RMSNorm to its row sums, and write the NEXT matvec's packed input (with the residual add and the
// norm weights folded in) or silu(gate) * up from its epilogue.
#pragma once

#include <cstdlib>
#include <mutex>

#include "qmm_gemv_device.cuh"
#include "qmm_kernels.h"
#include "qmm_pack.cuh"

namespace qmm {

namespace {

// Shared memory of one CTA, carved from the dynamic allocation:
//   slots  TILES*WARPS*DEPTH x (tile [+ batches 2..16: that chunk's activation record]) | mbarriers
//   (+1 for the activations) | (batch 1) all activation records + 512 zero bytes | cross-warp reduction
template <int FMT, int MC, int WARPS, int DEPTH, int TILES>
struct SmemPlan {
    static constexpr int NW = WARPS * TILES;
    static constexpr int XCHUNK = MC == 1 ? 0 : XSlot<Cols<MC>::NCP>::BYTES;
    static constexpr int SLOT = tile_bytes(FMT) + XCHUNK;
    static constexpr int SLOTS_BYTES = NW * DEPTH * SLOT;
    static constexpr int BAR_OFF = SLOTS_BYTES;
    static constexpr int BAR_BYTES = (((NW * DEPTH + 1) * 8 + 15) / 16) * 16;
    static constexpr int X_OFF = BAR_OFF + BAR_BYTES;
    __host__ __device__ static int x_bytes(int kc, int mc) { return mc == 1 ? (int)xpack1_bytes(kc) + 512 : 0; }
    __host__ __device__ static int red_off(int kc, int mc) { return X_OFF + x_bytes(kc, mc); }
    __host__ __device__ static int total(int kc, int mc) { return red_off(kc, mc) + NW * 16 * mc * 4; }
};

// WARPS warps share one row tile; a CTA holds TILES row tiles (2 for EPI_RESID_PACK: the 32 rows of
// one quantization block of the output, so the epilogue can quantize them without leaving the CTA).
// Registers decide how many CTAs an SM holds, and a batch-1 grid of 768 row tiles wants six CTAs of
// 256 threads on every SM at once (42 registers at most): the bound keeps the fp32-packing prologue
// and the fused epilogues from costing a second wave.
template <int MC, int THREADS, int EPI>
constexpr int gemv_min_blocks()
{
    return EPI == EPI_RESID_PACK ? 1 : EPI == EPI_SWIGLU_PACK ? 3 : MC > 1 ? 7 : (THREADS <= 256 ? 6 : 3);
}

template <int FMT, int MC, int WARPS, int DEPTH, int EPI, int TILES, bool XF32>
__global__ void __launch_bounds__(WARPS * TILES * 32, gemv_min_blocks<MC, WARPS * TILES * 32, EPI>())
    gemv_kernel(WeightView v, XPackView xp, float* __restrict__ y, int m, int* __restrict__ status, PeerScatter ps,
                GemvFuse fu)
{
    using Plan = SmemPlan<FMT, MC, WARPS, DEPTH, TILES>;
    constexpr int NW = WARPS * TILES;
    constexpr int NOUT = Cols<MC>::NOUT;
    constexpr uint32_t TILE = tile_bytes(FMT);
    static_assert(EPI == EPI_STORE || MC == 1, "fused epilogues exist for batch 1 only");
    static_assert(TILES == epi_tiles(EPI), "row tiles per CTA follow from the fused form");
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float s_in_sh;  // 1/rms factor of the input activations

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int wl = warp % WARPS;                                // this warp's place among its tile's warps
    const int64_t tile_row = (int64_t)blockIdx.x * TILES + warp / WARPS;  // row tile of this warp
    const int kc = v.kc;
    uint8_t* my_slots = smem + (size_t)warp * DEPTH * Plan::SLOT;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Plan::BAR_OFF);
    uint64_t* my_bars = bars + warp * DEPTH;
    uint64_t* xbar = bars + NW * DEPTH;
    const uint8_t* my_tiles = v.tiles + (size_t)tile_row * kc * TILE;
    const int n_my = (wl < kc && tile_row < v.rt) ? (kc - wl + WARPS - 1) / WARPS : 0;

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
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)(wl + s * WARPS) * TILE, TILE,
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
    // 2. everything below may read what earlier kernels in the stream produced
    pdl_wait();

    unsigned int epoch = 0;
    if constexpr (MC == 1 && (EPI == EPI_STORE || EPI == EPI_RESID_PACK)) {
        if (ps.n_peers > 0) {
            epoch = (unsigned int)(*ps.pos * ps.sites + ps.site + 1);
        }
    }
    XSrc<MC> xsrc;
    bool ok = true;
    float h_pre = 0.0f, w_pre = 0.0f;  // EPI_RESID_PACK: residual and norm weight of this thread's row
    if constexpr (MC == 1) {
        uint8_t* xbase = smem + Plan::X_OFF;
        const uint32_t xbytes = (uint32_t)xpack1_bytes(kc);
        if (!XF32 && threadIdx.x == 0) {  // the thread that initialised xbar
            mbar_expect_tx(xbar, xbytes);
            bulk_copy_g2s(xbase, xp.base, xbytes, xbar);
        }
        if (warp == NW - 1) {
            // the scalar RMSNorm factor of the input: the producer left one sum of squares per 32 activations
            double t = 0.0;
            if (fu.ss_in) {
                for (int i = lane; i < fu.ss_count; i += 32) {
                    t += fu.ss_in[i];
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
                }
            }
            if (lane == 0) {
                s_in_sh = fu.ss_in ? (float)(1.0 / sqrt(t / (double)fu.d_in + (double)fu.eps)) : 1.0f;
            }
        }
        if constexpr (EPI == EPI_RESID_PACK) {
            if (threadIdx.x < 32) {
                const int64_t row = (int64_t)blockIdx.x * 32 + threadIdx.x;
                if (row < v.n) {
                    h_pre = fu.h_in[row];
                    w_pre = fu.norm_w[row];
                }
            }
        }
        if constexpr (XF32) {
            // pack the fp32 activations here: spans of 128, one float4 per lane, all loads of a thread issued
            // before the first is used.  Every CTA reads the same few KB: each starts at another span, so
            // that the CTAs do not all ask the same L2 lines at the same moment.
            const int nspan = (int)(v.k / 128);
            constexpr int MAXS = 4;
            const int rot = nspan > 0 ? (int)((blockIdx.x * 13u) % (unsigned)nspan) : 0;
            const float* xsrc_f = fu.x_f32;
            for (int s0 = warp; s0 < nspan; s0 += NW * MAXS) {
                float4 xv[MAXS];
#pragma unroll
                for (int i = 0; i < MAXS; ++i) {
                    const int sq = s0 + i * NW;
                    if (sq < nspan) {
                        const int sp = sq + rot < nspan ? sq + rot : sq + rot - nspan;
                        xv[i] = __ldcg(reinterpret_cast<const float4*>(xsrc_f) + sp * 32 + lane);
                    }
                }
#pragma unroll
                for (int i = 0; i < MAXS; ++i) {
                    const int sq = s0 + i * NW;
                    if (sq < nspan) {
                        const int sp = sq + rot < nspan ? sq + rot : sq + rot - nspan;
                        warp_pack_span128(xv[i], xbase + (size_t)(sp >> 1) * XPK1_REC, (sp & 1) * 4);
                    }
                }
            }
            for (int blk = nspan * 4 + warp; blk < kc * 8; blk += NW) {  // the ragged end, then zero blocks
                const int64_t e = (int64_t)blk * 32 + lane;
                warp_pack_block32(e < v.k ? __ldcg(xsrc_f + e) : 0.0f, xbase + (size_t)(blk >> 3) * XPK1_REC, blk & 7);
            }
        }
        __syncthreads();  // xbar initialised, zero page written, activations packed
        xsrc.base = xbase;
        xsrc.zeros = xbase + xbytes;
        if (!XF32 && !mbar_wait(xbar, 0)) {
            ok = false;
            if (lane == 0) {
                atomicExch(status, 2);
            }
        }
    } else {
        if (threadIdx.x == 0) {
            s_in_sh = 1.0f;
        }
        xsrc.base = nullptr;
        if (lane == 0) {
            for (int s = 0; s < DEPTH && s < n_my; ++s) {
                uint64_t* bar = &my_bars[s];
                mbar_expect_tx(bar, Plan::XCHUNK);
                bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT + TILE, xp.base + (size_t)(wl + s * WARPS) * Plan::XCHUNK,
                              Plan::XCHUNK, bar);
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
                compute_chunk_m1<FMT>(my_slots + (size_t)s * Plan::SLOT, xsrc, wl + i * WARPS, lane, acc);
            } else {
                xsrc.attach(my_slots + (size_t)s * Plan::SLOT + TILE);
                compute_chunk<FMT, MC>(my_slots + (size_t)s * Plan::SLOT, xsrc, lane, acc);
            }
        }
        __syncwarp();
        if (ok && lane == 0 && i + DEPTH < n_my) {
            fence_proxy_async();  // order this warp's reads of the slot before the refill
            const int cn = wl + (i + DEPTH) * WARPS;
            mbar_expect_tx(&my_bars[s], TILE);
            bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT, my_tiles + (size_t)cn * TILE, TILE, &my_bars[s]);
            if constexpr (MC > 1) {
                mbar_expect_tx(&my_bars[s], Plan::XCHUNK);
                bulk_copy_g2s(my_slots + (size_t)s * Plan::SLOT + TILE, xp.base + (size_t)cn * Plan::XCHUNK, Plan::XCHUNK,
                              &my_bars[s]);
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
    const float s_in = s_in_sh;

    if constexpr (EPI == EPI_STORE) {
        for (int i = threadIdx.x; i < 16 * MC; i += NW * 32) {
            const int col = i >> 4;
            const int r = i & 15;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                sum += red[(w * 16 + r) * MC + col];
            }
            sum *= s_in;
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
    } else if constexpr (EPI == EPI_RESID_PACK) {
        if (warp == 0) {  // lane = row within the CTA's 32 rows: warps lane/16*WARPS .. +WARPS-1 hold its partial sums
            float sum = 0.0f;
            const int w0 = (lane >> 4) * WARPS, r = lane & 15;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                sum += red[(w0 + w) * 16 + r];
            }
            sum *= s_in;
            const int64_t row = (int64_t)blockIdx.x * 32 + lane;
            if (ps.n_peers > 0 && row < v.n) {
                // tensor parallelism: this rank's partial goes to every peer, the peers' partials are awaited
#pragma unroll
                for (int p = 0; p < QMM_MAX_PEERS; ++p) {
                    if (p < ps.n_peers) {
                        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(ps.dst[p] + row),
                                     "r"(__float_as_uint(sum)), "r"(epoch)
                                     : "memory");
                    }
                }
                bool waiting = *reinterpret_cast<volatile int*>(ps.wait_status) == 0;
                float total = 0.0f;
                for (int r = 0; r < ps.tp_size; ++r) {
                    if (r == ps.tp_rank) {
                        total += sum;
                        continue;
                    }
                    const uint2* src = ps.recv + (size_t)r * v.n + row;
                    uint2 pk;
                    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(pk.x), "=r"(pk.y) : "l"(src) : "memory");
                    unsigned int spin = 0;
                    while (waiting && pk.y != epoch) {
                        if (++spin > ps.spin_limit) {
                            waiting = false;
                            atomicExch(ps.wait_status, 5);  // a peer's addend never came; the sum is incomplete
                            break;
                        }
                        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];"
                                     : "=r"(pk.x), "=r"(pk.y)
                                     : "l"(src)
                                     : "memory");
                    }
                    total += __uint_as_float(pk.x);
                }
                sum = total;
            }
            const float hv = h_pre + sum;
            if (row < v.n) {
                fu.h_out[row] = hv;
                if (y) {
                    y[row] = sum;
                }
            }
            double sq = (double)hv * (double)hv;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
            }
            if (lane == 0) {
                fu.ss_out[blockIdx.x] = sq;
            }
            warp_pack_block32(hv * w_pre, fu.packed_out + (size_t)(blockIdx.x >> 3) * XPK1_REC, blockIdx.x & 7);
        }
    } else if constexpr (EPI == EPI_SWIGLU_PACK) {
        if (warp == 0) {  // lane = channel within the CTA's 32: row tile lane / 8, tile rows lane % 8 (gate) and + 8 (up)
            const int w0 = (lane >> 3) * WARPS, r = lane & 7;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                gate += red[(w0 + w) * 16 + r];
                up += red[(w0 + w) * 16 + r + 8];
            }
            gate *= s_in;
            up *= s_in;
            const int64_t ch = (int64_t)blockIdx.x * 32 + lane;
            const float act = 2 * ch < v.n ? (gate * (1.0f / (1.0f + expf(-gate)))) * up : 0.0f;
            if (y && 2 * ch < v.n) {
                y[ch] = act;
            }
            warp_pack_block32(act, fu.packed_out + (size_t)(blockIdx.x >> 3) * XPK1_REC, blockIdx.x & 7);
        }
    } else {
        if (threadIdx.x < 8) {
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                gate += red[w * 16 + threadIdx.x];
                up += red[w * 16 + threadIdx.x + 8];
            }
            gate *= s_in;
            up *= s_in;
            const int64_t ch = (int64_t)blockIdx.x * 8 + threadIdx.x;
            if (2 * ch < v.n) {
                // sigmoid = 1 / (1 + exp(-x)), SiLU = x * sigmoid(x) (src/LiteNN/Layer/Activation.h:20-33,52-59)
                y[ch] = (gate * (1.0f / (1.0f + expf(-gate)))) * up;
            }
        }
    }
}

// Ring depth per format: 28-37 KB of tiles in flight per CTA.
template <int FMT>
struct Tune {
    static constexpr int WARPS = 4;
    static constexpr int DEPTH = FMT == FMT_Q8_0 ? 2 : 3;
};

template <int FMT, int MC, int WARPS, int DEPTH, int EPI, bool XF32>
cudaError_t launch_gemv_xsrc(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                             const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream)
{
    constexpr int TILES = epi_tiles(EPI);
    using Plan = SmemPlan<FMT, MC, WARPS, DEPTH, TILES>;
    auto kernel = gemv_kernel<FMT, MC, WARPS, DEPTH, EPI, TILES, XF32>;
    int smem = Plan::total(w.kc, MC);
    if (smem > 227 * 1024) {
        return cudaErrorInvalidConfiguration;
    }
    if (w.rt % TILES != 0) {
        return cudaErrorInvalidValue;
    }
    const int grid = w.rt / TILES;
    // Residency cap.  The block scheduler fills an SM up to its limit before it is even with the others, so
    // a grid of 688 CTAs that could sit 7 to an SM leaves a third of the SMs with little to do (measured on
    // B200: 6.7 us at a limit of 7, 5.2 us at 5 for W[11008,4096]).  The dynamic shared memory request is
    // padded so that no SM can hold more than its even share, ceil(grid / SMs), of the CTAs.
    static std::mutex mu;
    static int sm_count[64] = {};
    static int configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && sm_count[dev] == 0) {
            cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        }
        int share = dev >= 0 && dev < 64 && sm_count[dev] > 0 ? (grid + sm_count[dev] - 1) / sm_count[dev] : 0;
        if (const char* env = getenv("QMM_GEMV_CTAS_PER_SM")) {  // tuning aid
            share = atoi(env);
        }
        if (share >= 1 && share <= 16) {
            const int want = 232448 / share - 1024 - 256;
            smem = want > smem ? want : smem;
        }
        // the opt-in limit is a per-device function attribute; raise it only when needed
        if (dev < 0 || dev >= 64 || configured[dev] < smem) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) {
                return e;
            }
            if (dev >= 0 && dev < 64) {
                configured[dev] = smem;
            }
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(WARPS * TILES * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, kernel, w, xp, y, m, status, ps, fu);
}

template <int FMT, int MC, int WARPS, int DEPTH, int EPI>
cudaError_t launch_gemv_variant(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                                const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream)
{
    if constexpr (MC == 1 && EPI != EPI_SWIGLU && EPI != EPI_SWIGLU_PACK) {
        if (fu.x_f32 != nullptr) {
            return launch_gemv_xsrc<FMT, MC, WARPS, DEPTH, EPI, true>(w, xp, y, m, status, ps, fu, stream);
        }
    }
    if (fu.x_f32 != nullptr) {
        return cudaErrorInvalidValue;
    }
    return launch_gemv_xsrc<FMT, MC, WARPS, DEPTH, EPI, false>(w, xp, y, m, status, ps, fu, stream);
}

// Batch 1: warps x ring slots by row length.
//   K of 2304..4096: eight warps with one slot each (the whole row tile is requested by the first
//   instruction, 18 KB per CTA) measured faster than four warps with three slots for every format but
//   Q8_0, whose larger tiles would leave fewer CTAs per SM.
//   K > 4096: with four warps a warp would walk 6-28 tiles one after the other, and in a chain of
//   dependent matvecs that walk starts only when the activations arrive; more warps per row tile
//   shorten it, as long as two CTAs still fit on an SM.
template <int FMT, int EPI>
cudaError_t launch_gemv_m1(const WeightView& w, const XPackView& xp, float* y, int* status, const PeerScatter& ps,
                           const GemvFuse& fu, cudaStream_t stream)
{
    constexpr int TILES = epi_tiles(EPI);
    constexpr int LIMIT = 113 * 1024;
    if constexpr (TILES == 2) {
        // The residual form has two row tiles per CTA and n / 32 CTAs: 128 for a 4096-wide model, 256 for an
        // 8192-wide one.  All of them should be resident at once (a second wave of a few CTAs doubles the
        // kernel's time), so the variant is the deepest one whose shared memory lets ceil(CTAs / SMs) CTAs
        // share an SM.  8 warps per tile with three slots each walk a long row with 110 KB in flight per CTA
        // (ffn_down of the 7B shape, K = 11008: 7.1 us against 8.1 us with 16 warps x 2 slots).
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) {
            return cudaErrorInvalidDevice;
        }
        const int ctas = w.rt / 2;
        const int per_sm = (ctas + sms - 1) / sms;
        const int budget = 232448 / per_sm - 1280;
        if (w.kc > 8 && w.kc <= 16 && FMT != FMT_Q8_0 && SmemPlan<FMT, 1, 8, 1, 2>::total(w.kc, 1) <= budget) {
            return launch_gemv_variant<FMT, 1, 8, 1, EPI>(w, xp, y, 1, status, ps, fu, stream);
        }
        if (w.kc > 16 && SmemPlan<FMT, 1, 8, 3, 2>::total(w.kc, 1) <= budget) {
            return launch_gemv_variant<FMT, 1, 8, 3, EPI>(w, xp, y, 1, status, ps, fu, stream);
        }
        if (SmemPlan<FMT, 1, 4, 3, 2>::total(w.kc, 1) <= budget) {
            return launch_gemv_variant<FMT, 1, 4, 3, EPI>(w, xp, y, 1, status, ps, fu, stream);
        }
        if (SmemPlan<FMT, 1, 4, 2, 2>::total(w.kc, 1) <= budget) {
            return launch_gemv_variant<FMT, 1, 4, 2, EPI>(w, xp, y, 1, status, ps, fu, stream);
        }
        // more than one CTA per SM wanted and nothing deeper fits: one slot per warp, the number of CTAs keeps
        // the bytes in flight up
        return launch_gemv_variant<FMT, 1, 4, 1, EPI>(w, xp, y, 1, status, ps, fu, stream);
    }
    if (w.kc > 8 && w.kc <= 16 && FMT != FMT_Q8_0) {
        return launch_gemv_variant<FMT, 1, 8, 1, EPI>(w, xp, y, 1, status, ps, fu, stream);
    }
    if (w.kc > 32 && SmemPlan<FMT, 1, 16, 2, 1>::total(w.kc, 1) <= LIMIT) {
        return launch_gemv_variant<FMT, 1, 16, 2, EPI>(w, xp, y, 1, status, ps, fu, stream);
    }
    if (w.kc > 16 && SmemPlan<FMT, 1, 8, 3, TILES>::total(w.kc, 1) <= LIMIT) {
        return launch_gemv_variant<FMT, 1, 8, 3, EPI>(w, xp, y, 1, status, ps, fu, stream);
    }
    return launch_gemv_variant<FMT, 1, Tune<FMT>::WARPS, Tune<FMT>::DEPTH, EPI>(w, xp, y, 1, status, ps, fu, stream);
}

template <int FMT, int MC>
cudaError_t launch_gemv_batch(const WeightView& w, const XPackView& xp, float* y, int m, int* status, cudaStream_t stream)
{
    // batches 2..16 carry 3-10 KB of activations per slot: a shallower ring keeps 2-3 CTAs per SM
    constexpr int DEPTH = MC == 4 && FMT != FMT_Q8_0 ? 3 : 2;
    const PeerScatter none = {};
    const GemvFuse plain = {};
    return launch_gemv_variant<FMT, MC, Tune<FMT>::WARPS, DEPTH, EPI_STORE>(w, xp, y, m, status, none, plain, stream);
}

template <int FMT>
cudaError_t launch_gemv_fmt(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                            const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream)
{
    if (m == 1) {
        switch (fu.mode) {
        case EPI_STORE: return launch_gemv_m1<FMT, EPI_STORE>(w, xp, y, status, ps, fu, stream);
        case EPI_RESID_PACK: return launch_gemv_m1<FMT, EPI_RESID_PACK>(w, xp, y, status, ps, fu, stream);
        case EPI_SWIGLU: return launch_gemv_m1<FMT, EPI_SWIGLU>(w, xp, y, status, ps, fu, stream);
        // four row tiles per CTA, two warps per tile with three slots each: 8 warps walk kc / 2 tiles apiece
        // (8 for K = 4096) and a third of a 1376-tile gate|up weight's CTAs fit an SM together
        case EPI_SWIGLU_PACK: return launch_gemv_variant<FMT, 1, 2, 3, EPI_SWIGLU_PACK>(w, xp, y, 1, status, ps, fu, stream);
        default: return cudaErrorInvalidValue;
        }
    }
    if (fu.mode != EPI_STORE || fu.ss_in != nullptr || fu.x_f32 != nullptr || ps.n_peers > 0) {
        return cudaErrorInvalidValue;
    }
    if (m <= 4) {
        return launch_gemv_batch<FMT, 4>(w, xp, y, m, status, stream);
    }
    if (m <= 8) {
        return launch_gemv_batch<FMT, 8>(w, xp, y, m, status, stream);
    }
    if (m <= 12) {
        return launch_gemv_batch<FMT, 12>(w, xp, y, m, status, stream);
    }
    return launch_gemv_batch<FMT, 16>(w, xp, y, m, status, stream);
}

}  // namespace

}  // namespace qmm

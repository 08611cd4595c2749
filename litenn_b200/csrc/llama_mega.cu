// Persistent decoder kernel: one cooperative launch runs a whole token of the decoder
// (tools/gguf/LLaMABuilder.cpp:568-668 per block, :719-733 logits) on one CTA per SM.
//
// Why one kernel: a decode step is a chain of ~9 dependent small operators per block; as
// separate launches each link costs a few microseconds during which HBM idles, although the
// only large traffic — the quantized weights — never depends on the chain.  Here every warp owns
// a small ring of shared-memory slots and walks its own, statically known sequence of weight
// tiles across ALL linears of the token, refilling a slot with a TMA bulk copy the moment it
// has been read.  The copies therefore run ahead of the dependency chain (through grid
// barriers, attention and norms) and HBM stays busy while the chain catches up.
//
// Work split.  A linear's 16-row tiles are dealt round-robin to groups of `wpr` warps
// (MEGA_WARPS / wpr groups per CTA); the warps of a group split the 256-column chunks of a row
// tile, multiply them exactly as the stand-alone matvec does (qmm_gemv_device.cuh) and add
// their partial sums in shared memory in a fixed order.  Between linears the CTAs meet at a
// grid barrier (bounded spin on an arrival counter).  What sits between two linears is
// recomputed by every CTA from the previous linear's output in L2 — residual add + RMSNorm,
// merge of the attention partials, SwiGLU — and quantized straight into the CTA's shared
// memory; each CTA keeps its own copy of the residual stream there.  Attention runs as its
// own stage: CTA = (head, key split), 24 warps over the split's keys, cached keys preloaded
// before the barrier that precedes it.
//
// Every wait is bounded; when one runs out the CTA records a status, stops waiting anywhere,
// drains its outstanding copies and leaves, and the host reports QMM_E_KERNEL.
#include "llama_device.cuh"
#include "llama_kernels.h"
#include "qmm_gemv_device.cuh"
#include "qmm_layout.cuh"

namespace qmm {

namespace {

constexpr int MEGA_THREADS = MEGA_WARPS * 32;
constexpr int MEGA_MAX_SLOTS = 3;

// ---- shared memory plan ----------------------------------------------------------------------
struct MegaSmem {
    int ring, bars, table, zeros, xpack, hres, red, dred, flag, total;
    __host__ __device__ MegaSmem(int d_model, int hd, int kc_max, int n_lin)
    {
        int o = 0;
        ring = o;
        o += MEGA_WARPS * MEGA_RING_BYTES;
        bars = o;
        o += MEGA_WARPS * MEGA_MAX_SLOTS * 8;
        table = o;  // the MegaLinear table of the model
        o += (n_lin * (int)sizeof(MegaLinear) + 15) / 16 * 16;
        zeros = o;  // 512 zero bytes for the MMA lanes that carry no activation
        o += 512;
        xpack = o;  // packed activations of the current linear; attention scratch in its stage
        int xb = (int)xpack1_bytes(kc_max);
        const int attn = MEGA_WARPS * (hd + 2) * 4;
        xb = xb > attn ? xb : attn;
        o += (xb + 15) / 16 * 16;
        hres = o;  // residual stream, fp32
        o += d_model * 4;
        red = o;  // [2][MEGA_WARPS][16] partial row sums
        o += 2 * MEGA_WARPS * 16 * 4;
        dred = o;  // [MEGA_WARPS] doubles
        o = (o + 7) / 8 * 8;
        dred = o;
        o += (MEGA_WARPS + 1) * 8;
        flag = o;
        o += 16;
        total = o;
    }
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void group_barrier(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Grid-wide barrier: every CTA adds one arrival, thread 0 spins (bounded) until all of this
// round's arrivals are in.  `target` lives in thread 0.  Returns false once anything failed.
__device__ __forceinline__ bool grid_barrier(const MegaArgs& a, unsigned int& target, int* s_flag, bool ok)
{
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (threadIdx.x == 0) {
        target += gridDim.x;
        __threadfence();
        atomicAdd(a.sync, 1u);
        bool good = ok;
        if (good) {
            unsigned int spins = 0;
            while ((int)(ld_acquire_gpu(a.sync) - target) < 0) {
                ++spins;
                if ((spins & 255u) == 0u && *reinterpret_cast<volatile int*>(a.status) != 0) {
                    good = false;  // another CTA gave up
                    break;
                }
                if (spins > (1u << 21)) {
                    atomicExch(a.status, 3);
                    good = false;
                    break;
                }
            }
        }
        __threadfence();
        *s_flag = good ? 1 : 0;
    }
    __syncthreads();
    return *s_flag != 0;
}

// ---- the per-warp tile stream -------------------------------------------------------------------

// Where a warp's prefetch stands in its sequence: linear s, row tile r, chunk c.
struct TileCursor {
    int s, r, c;
    int rt, kc, wpr, stride;
    const uint8_t* tiles;
    uint32_t tb;
    bool valid;
};

__device__ __forceinline__ void cursor_enter(TileCursor& cu, const MegaLinear* lin, int n_lin, int warp)
{
    while (cu.s < n_lin) {
        const MegaLinear& d = lin[cu.s];
        const int wpr = d.wpr;
        const int r0 = (warp / wpr) * gridDim.x + blockIdx.x;
        if (r0 < d.rt && (warp % wpr) < d.kc) {
            cu.r = r0;
            cu.c = warp % wpr;
            cu.rt = d.rt;
            cu.kc = d.kc;
            cu.wpr = wpr;
            cu.stride = (MEGA_WARPS / wpr) * gridDim.x;
            cu.tiles = d.tiles;
            cu.tb = d.tile_bytes;
            cu.valid = true;
            return;
        }
        ++cu.s;
    }
    cu.valid = false;
}

__device__ __forceinline__ void cursor_advance(TileCursor& cu, const MegaLinear* lin, int n_lin, int warp)
{
    cu.c += cu.wpr;
    if (cu.c < cu.kc) {
        return;
    }
    cu.c = warp % cu.wpr;
    cu.r += cu.stride;
    if (cu.r < cu.rt) {
        return;
    }
    ++cu.s;
    cursor_enter(cu, lin, n_lin, warp);
}

// Ring of one warp.  Slots are tile-sized, so a run of tiles of another size starts only when
// the ring has drained; both ends then restart at slot 0.
struct Ring {
    uint8_t* base;
    uint64_t* bars;
    uint32_t tb;       // tile bytes of the current run
    int ns;            // slots of the current run
    int qi, qc;        // next slot to fill / to read
    uint32_t phase;    // bit s: parity the next wait on slot s expects
    unsigned int issued, consumed;
};

__device__ __forceinline__ void ring_fill(Ring& rg, TileCursor& pf, const MegaLinear* lin, int n_lin, int warp,
                                          int lane)
{
    while (pf.valid) {
        if (pf.tb != rg.tb) {
            if (rg.issued != rg.consumed) {
                break;
            }
            rg.tb = pf.tb;
            const int fit = MEGA_RING_BYTES / (int)pf.tb;
            rg.ns = fit < MEGA_MAX_SLOTS ? fit : MEGA_MAX_SLOTS;
            rg.qi = 0;
            rg.qc = 0;
        }
        if ((int)(rg.issued - rg.consumed) >= rg.ns) {
            break;
        }
        if (lane == 0) {
            uint64_t* bar = rg.bars + rg.qi;
            mbar_expect_tx(bar, rg.tb);
            bulk_copy_g2s(rg.base + (size_t)rg.qi * rg.tb, pf.tiles + ((size_t)pf.r * pf.kc + pf.c) * rg.tb, rg.tb, bar);
        }
        rg.qi = rg.qi + 1 == rg.ns ? 0 : rg.qi + 1;
        ++rg.issued;
        cursor_advance(pf, lin, n_lin, warp);
    }
}

// Waits for the next tile of the ring; returns its address (nullptr after a timeout).
__device__ __forceinline__ const uint8_t* ring_acquire(Ring& rg, bool& ok, int* status, int lane)
{
    if (!ok) {
        return rg.base;
    }
    if (!mbar_wait(rg.bars + rg.qc, (rg.phase >> rg.qc) & 1u)) {
        ok = false;
        if (lane == 0) {
            atomicExch(status, 1);
        }
        return rg.base;  // the slot stays outstanding for the drain
    }
    rg.phase ^= 1u << rg.qc;
    return rg.base + (size_t)rg.qc * rg.tb;
}

__device__ __forceinline__ void ring_release(Ring& rg, bool ok, int lane)
{
    __syncwarp();
    if (!ok) {
        return;  // after a timeout nothing more is issued; the drain at the end takes over
    }
    if (lane == 0) {
        fence_proxy_async();  // this warp's reads of the slot come before the refill
    }
    rg.qc = rg.qc + 1 == rg.ns ? 0 : rg.qc + 1;
    ++rg.consumed;
}

// ---- one linear ---------------------------------------------------------------------------------

struct Warp {
    int warp, lane;
    Ring ring;
    TileCursor pf;
    bool ok;
};

template <int FMT>
__device__ __forceinline__ void linear_rows(const MegaArgs& a, const MegaLinear* lin, const MegaLinear& d, Warp& w,
                                            const XShared& xs, float* red)
{
    const int n_lin = 4 * a.n_layers + 1;
    const int wpr = d.wpr, g = w.warp / wpr, wi = w.warp % wpr;
    const int stride = (MEGA_WARPS / wpr) * gridDim.x;
    const int lg = w.lane >> 2, lt = w.lane & 3;
    int parity = 0;
    for (int r = g * gridDim.x + blockIdx.x; r < d.rt; r += stride) {
        float acc[2] = {0.0f, 0.0f};
        for (int c = wi; c < d.kc; c += wpr) {
            const uint8_t* slot = ring_acquire(w.ring, w.ok, a.status, w.lane);
            if (w.ok) {
                compute_chunk_m1<FMT>(slot, xs, c, w.lane, acc);
            }
            ring_release(w.ring, w.ok, w.lane);
            if (w.ok) {
                ring_fill(w.ring, w.pf, lin, n_lin, w.warp, w.lane);
            }
        }
        // lanes t=0 and t=1 each folded one block of every pair
        acc[0] += __shfl_xor_sync(0xFFFFFFFFu, acc[0], 1);
        acc[1] += __shfl_xor_sync(0xFFFFFFFFu, acc[1], 1);
        float* mine = red + (parity * MEGA_WARPS + w.warp) * 16;
        if (lt == 0) {
            mine[lg] = acc[0];
            mine[lg + 8] = acc[1];
        }
        group_barrier(1 + g, wpr * 32);
        if (wi == 0 && w.lane < 16) {
            const float* grp = red + (parity * MEGA_WARPS + g * wpr) * 16 + w.lane;
            float sum = 0.0f;
            for (int j = 0; j < wpr; ++j) {
                sum += grp[j * 16];
            }
            const int row = r * 16 + w.lane;
            if (row < d.n) {
                d.y[row] = sum;
            }
        }
        parity ^= 1;
    }
}

__device__ __forceinline__ void run_linear(const MegaArgs& a, int s, Warp& w, uint8_t* smem, const MegaSmem& sm)
{
    const MegaLinear* lin = reinterpret_cast<const MegaLinear*>(smem + sm.table);
    const MegaLinear d = lin[s];
    XShared xs;
    const uint8_t* xp = smem + sm.xpack;
    xs.xq = xp;
    xs.xs = reinterpret_cast<const float*>(xp + xpack1_xs_offset(d.kc));
    xs.xsum = reinterpret_cast<const int2*>(xp + xpack1_xsum_offset(d.kc));
    xs.zeros = smem + sm.zeros;
    xs.cur = xp;
    float* red = reinterpret_cast<float*>(smem + sm.red);
    switch (d.fmt) {
    case FMT_Q4_0: linear_rows<FMT_Q4_0>(a, lin, d, w, xs, red); break;
    case FMT_Q8_0: linear_rows<FMT_Q8_0>(a, lin, d, w, xs, red); break;
    case FMT_Q4_K: linear_rows<FMT_Q4_K>(a, lin, d, w, xs, red); break;
    default: linear_rows<FMT_Q6_K>(a, lin, d, w, xs, red); break;
    }
}

// ---- what sits between the linears --------------------------------------------------------------

// Sum over the CTA of one double per warp-reduced lane; every thread gets the total.
// Only warp 0 adds the per-warp values, so the double-precision pipe sees 32 threads, not 768.
__device__ __forceinline__ double cta_sum_double(double v, double* dred, int warp, int lane)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    }
    if (lane == 0) {
        dred[warp] = v;
    }
    __syncthreads();
    if (warp == 0) {
        double t = lane < MEGA_WARPS ? dred[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
        }
        if (lane == 0) {
            dred[MEGA_WARPS] = t;
        }
    }
    __syncthreads();
    return dred[MEGA_WARPS];
}

// hres = dequantized row `token` of the embedding payload (the first linear's residual input).
__device__ __noinline__ void stage_embed(const MegaArgs& a, uint8_t* smem, const MegaSmem& sm)
{
    float* hres = reinterpret_cast<float*>(smem + sm.hres);
    const int d = a.d_model;
    const int belems = block_elems(a.embd_fmt), bbytes = block_bytes(a.embd_fmt);
    const uint8_t* erow = a.embd + (int64_t)(*a.token) * (d / belems) * bbytes;
    for (int idx = threadIdx.x; idx < d; idx += MEGA_THREADS) {
        hres[idx] = dequant_raw_element(a.embd_fmt, erow + (idx / belems) * bbytes, idx % belems);
    }
    __syncthreads();
}

// hres += add (when given); packed = pack(rmsnorm(hres) * nw).  Every CTA does the whole row;
// lane L of the warp that owns chunk c holds elements 8L..8L+7 (d is a multiple of 32, so a
// lane's eight elements are all inside or all outside the row).
__device__ __noinline__ void stage_norm(const MegaArgs& a, const float* add, const float* nw, int kc, int warp,
                                        int lane, uint8_t* smem, const MegaSmem& sm)
{
    constexpr int MAXC = 2;  // chunks per warp kept in registers (d_model <= 2 * 256 * MEGA_WARPS)
    float* hres = reinterpret_cast<float*>(smem + sm.hres);
    const int d = a.d_model;
    float4 av[MAXC][2], wv[MAXC][2];
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
        const int idx = (warp + j * MEGA_WARPS) * 256 + 8 * lane;
        const bool live = idx < d;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            av[j][q] = live && add ? __ldcg(reinterpret_cast<const float4*>(add + idx) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            wv[j][q] = live ? __ldg(reinterpret_cast<const float4*>(nw + idx) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    double ss = 0.0;
    float hv[MAXC][8];
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
        const int idx = (warp + j * MEGA_WARPS) * 256 + 8 * lane;
        if (idx < d) {
            const float4 h0 = *reinterpret_cast<const float4*>(hres + idx);
            const float4 h1 = *reinterpret_cast<const float4*>(hres + idx + 4);
            hv[j][0] = h0.x + av[j][0].x;
            hv[j][1] = h0.y + av[j][0].y;
            hv[j][2] = h0.z + av[j][0].z;
            hv[j][3] = h0.w + av[j][0].w;
            hv[j][4] = h1.x + av[j][1].x;
            hv[j][5] = h1.y + av[j][1].y;
            hv[j][6] = h1.z + av[j][1].z;
            hv[j][7] = h1.w + av[j][1].w;
            *reinterpret_cast<float4*>(hres + idx) = make_float4(hv[j][0], hv[j][1], hv[j][2], hv[j][3]);
            *reinterpret_cast<float4*>(hres + idx + 4) = make_float4(hv[j][4], hv[j][5], hv[j][6], hv[j][7]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                ss += (double)hv[j][i] * (double)hv[j][i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                hv[j][i] = 0.0f;
            }
        }
    }
    ss = cta_sum_double(ss, reinterpret_cast<double*>(smem + sm.dred), warp, lane);
    const double inv = 1.0 / sqrt(ss / (double)d + (double)a.eps);
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
        const int c = warp + j * MEGA_WARPS;
        if (c < kc) {
            float v[8];
            const float wl[8] = {wv[j][0].x, wv[j][0].y, wv[j][0].z, wv[j][0].w, wv[j][1].x, wv[j][1].y, wv[j][1].z, wv[j][1].w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = (float)((double)hv[j][i] * inv) * wl[i];
            }
            warp_pack_chunk(v, c, kc, smem + sm.xpack);
        }
    }
    __syncthreads();
}

// packed = pack(ctx), ctx = the attention partials of every head merged over the key splits.
// Partial rows are [max, sum, -, -, acc[hd]] (16-byte aligned).
__device__ __noinline__ void stage_ctx(const MegaArgs& a, int kc, int warp, int lane, uint8_t* smem, const MegaSmem& sm)
{
    const int hd = a.hd, ns = a.nsplit, width = a.n_heads * hd, row = hd + 4;
    for (int c = warp; c < kc; c += MEGA_WARPS) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = 0.0f;
        }
        const int idx0 = c * 256 + 8 * lane;  // 8 elements of one head (hd is a multiple of 8)
        if (idx0 < width) {
            const int head = idx0 / hd, e = idx0 % hd;
            const float* p = a.part + (int64_t)head * ns * row;
            float M = -INFINITY, L = 0.0f;
            for (int s0 = 0; s0 < ns; s0 += 4) {
                float2 ml[4];
                float4 x0[4], x1[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {  // all loads of four splits before any use
                    const int s2 = min(s0 + j, ns - 1);
                    ml[j] = __ldcg(reinterpret_cast<const float2*>(p + s2 * row));
                    x0[j] = __ldcg(reinterpret_cast<const float4*>(p + s2 * row + 4 + e));
                    x1[j] = __ldcg(reinterpret_cast<const float4*>(p + s2 * row + 8 + e));
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (s0 + j < ns && ml[j].x != -INFINITY) {
                        const float mn = fmaxf(M, ml[j].x);
                        const float fo = __expf(M - mn), fn = __expf(ml[j].x - mn);
                        L = L * fo + ml[j].y * fn;
                        v[0] = v[0] * fo + x0[j].x * fn;
                        v[1] = v[1] * fo + x0[j].y * fn;
                        v[2] = v[2] * fo + x0[j].z * fn;
                        v[3] = v[3] * fo + x0[j].w * fn;
                        v[4] = v[4] * fo + x1[j].x * fn;
                        v[5] = v[5] * fo + x1[j].y * fn;
                        v[6] = v[6] * fo + x1[j].z * fn;
                        v[7] = v[7] * fo + x1[j].w * fn;
                        M = mn;
                    }
                }
            }
            const float rl = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] *= rl;
            }
        }
        warp_pack_chunk(v, c, kc, smem + sm.xpack);
    }
    __syncthreads();
}

// packed = pack(silu(gate) * up) from gu = [gate | up]; ffn is a multiple of 32.
__device__ __noinline__ void stage_swiglu(const MegaArgs& a, const float* gu, int kc, int warp, int lane,
                                          uint8_t* smem, const MegaSmem& sm)
{
    const int ffn = a.ffn;
    for (int c0 = warp; c0 < kc; c0 += 2 * MEGA_WARPS) {
        float4 g[2][2], u[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {  // both chunks' loads before any use
            const int idx = (c0 + j * MEGA_WARPS) * 256 + 8 * lane;
            const bool live = idx < ffn;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                g[j][q] = live ? __ldcg(reinterpret_cast<const float4*>(gu + idx) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
                u[j][q] = live ? __ldcg(reinterpret_cast<const float4*>(gu + ffn + idx) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = c0 + j * MEGA_WARPS;
            if (c < kc) {
                const float gl[8] = {g[j][0].x, g[j][0].y, g[j][0].z, g[j][0].w, g[j][1].x, g[j][1].y, g[j][1].z, g[j][1].w};
                const float ul[8] = {u[j][0].x, u[j][0].y, u[j][0].z, u[j][0].w, u[j][1].x, u[j][1].y, u[j][1].z, u[j][1].w};
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[i] = (gl[i] / (1.0f + expf(-gl[i]))) * ul[i];
                }
                warp_pack_chunk(v, c, kc, smem + sm.xpack);
            }
        }
    }
    __syncthreads();
}

// ---- attention stage ------------------------------------------------------------------------------

// Item = (head, key split); warp w of the CTA takes the w-th part of the split's cached keys.
__device__ __forceinline__ void attn_ranges(const MegaArgs& a, int item, int pos, int warp, int& head, int& split,
                                            int& k0, int& k1)
{
    head = item % a.n_heads;
    split = item / a.n_heads;
    const int per_s = (pos + a.nsplit - 1) / a.nsplit;
    const int s0 = min(pos, split * per_s), s1 = min(pos, s0 + per_s);
    const int per_w = (s1 - s0 + MEGA_WARPS - 1) / MEGA_WARPS;
    k0 = min(s1, s0 + warp * per_w);
    k1 = min(s1, k0 + per_w);
}

template <int DPL>
struct AttnPre {
    KvBatch<DPL> batch;       // first eight cached keys of this warp's range (first item of the CTA)
    float cs[DPL / 2], sn[DPL / 2];  // rotation factors of this lane's pairs at the current position
};

// Before the barrier that follows the qkv linear: everything that depends only on earlier tokens.
template <int DPL>
__device__ __forceinline__ void attn_preload(const MegaArgs& a, const MegaLayer& ly, int pos, const Warp& w,
                                             AttnPre<DPL>& pre)
{
    constexpr int hd = 32 * DPL;
#pragma unroll
    for (int j = 0; j < DPL / 2; ++j) {
        const int i = w.lane * (DPL / 2) + j;
        const bool rot = 2 * i < a.rope_dim;
        pre.cs[j] = rot ? a.rope_cos[(int64_t)pos * (a.rope_dim / 2) + i] : 1.0f;
        pre.sn[j] = rot ? a.rope_sin[(int64_t)pos * (a.rope_dim / 2) + i] : 0.0f;
    }
    if ((int)blockIdx.x < a.n_heads * a.nsplit) {
        int head, split, k0, k1;
        attn_ranges(a, blockIdx.x, pos, w.warp, head, split, k0, k1);
        const int kvh = head / (a.n_heads / a.n_kv);
        const __half* kb = ly.cache_k + (int64_t)kvh * a.max_seq * hd + w.lane * DPL;
        const __half* vb = ly.cache_v + (int64_t)kvh * a.max_seq * hd + w.lane * DPL;
        kv_batch_load<DPL>(pre.batch, kb, vb, k0, k1);
    }
}

template <int DPL>
__device__ __forceinline__ void attn_stage(const MegaArgs& a, const MegaLayer& ly, const float* qkv, int pos,
                                           const Warp& w, const AttnPre<DPL>& pre, uint8_t* smem, const MegaSmem& sm)
{
    constexpr int hd = 32 * DPL;
    float* parts = reinterpret_cast<float*>(smem + sm.xpack);  // [MEGA_WARPS][hd + 2]
    const int items = a.n_heads * a.nsplit;
    const int group = a.n_heads / a.n_kv;
    const float scale = rsqrtf((float)hd);
    bool first = true;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        int head, split, k0, k1;
        attn_ranges(a, item, pos, w.warp, head, split, k0, k1);
        const int kvh = head / group;
        const __half* kb = ly.cache_k + (int64_t)kvh * a.max_seq * hd + w.lane * DPL;
        const __half* vb = ly.cache_v + (int64_t)kvh * a.max_seq * hd + w.lane * DPL;
        const bool takes_new = split == a.nsplit - 1 && w.warp == MEGA_WARPS - 1;
        float2 qx[DPL / 2], kx[DPL / 2], vx[DPL / 2];
#pragma unroll
        for (int j = 0; j < DPL / 2; ++j) {
            qx[j] = __ldcg(reinterpret_cast<const float2*>(qkv + head * hd + w.lane * DPL + 2 * j));
            if (takes_new) {
                kx[j] = __ldcg(reinterpret_cast<const float2*>(qkv + (a.n_heads + kvh) * hd + w.lane * DPL + 2 * j));
                vx[j] = __ldcg(
                    reinterpret_cast<const float2*>(qkv + (a.n_heads + a.n_kv + kvh) * hd + w.lane * DPL + 2 * j));
            }
        }
        float qv[DPL], acc[DPL];
#pragma unroll
        for (int j = 0; j < DPL / 2; ++j) {
            const bool rot = 2 * (w.lane * (DPL / 2) + j) < a.rope_dim;
            const float2 x = qx[j];
            const float ra = rot ? __fsub_rn(__fmul_rn(x.x, pre.cs[j]), __fmul_rn(x.y, pre.sn[j])) : x.x;
            const float rb = rot ? __fadd_rn(__fmul_rn(x.x, pre.sn[j]), __fmul_rn(x.y, pre.cs[j])) : x.y;
            qv[2 * j] = ra * scale;
            qv[2 * j + 1] = rb * scale;
            acc[2 * j] = 0.0f;
            acc[2 * j + 1] = 0.0f;
        }
        float m = -INFINITY, l = 0.0f;
        int kbase = k0;
        if (first) {
            kv_batch_apply<DPL>(pre.batch, qv, k0, k1, m, l, acc);
            kbase = k0 + 8;
        }
        for (; kbase < k1; kbase += 8) {
            KvBatch<DPL> cur;
            kv_batch_load<DPL>(cur, kb, vb, kbase, k1);
            kv_batch_apply<DPL>(cur, qv, kbase, k1, m, l, acc);
        }
        if (takes_new) {  // the new position: key and value straight from the qkv vector, as the cache rounds them
            __half kn[DPL], vn[DPL];
#pragma unroll
            for (int j = 0; j < DPL / 2; ++j) {
                const bool rot = 2 * (w.lane * (DPL / 2) + j) < a.rope_dim;
                const float2 x = kx[j];
                const float ra = rot ? __fsub_rn(__fmul_rn(x.x, pre.cs[j]), __fmul_rn(x.y, pre.sn[j])) : x.x;
                const float rb = rot ? __fadd_rn(__fmul_rn(x.x, pre.sn[j]), __fmul_rn(x.y, pre.cs[j])) : x.y;
                kn[2 * j] = __float2half_rn(ra);
                kn[2 * j + 1] = __float2half_rn(rb);
                vn[2 * j] = __float2half_rn(vx[j].x);
                vn[2 * j + 1] = __float2half_rn(vx[j].y);
            }
            if (head % group == 0) {
                __half* kd = ly.cache_k + ((int64_t)kvh * a.max_seq + pos) * hd + w.lane * DPL;
                __half* vd = ly.cache_v + ((int64_t)kvh * a.max_seq + pos) * hd + w.lane * DPL;
#pragma unroll
                for (int i = 0; i < DPL; i += 2) {
                    *reinterpret_cast<__half2*>(kd + i) = *reinterpret_cast<const __half2*>(&kn[i]);
                    *reinterpret_cast<__half2*>(vd + i) = *reinterpret_cast<const __half2*>(&vn[i]);
                }
            }
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                dot += qv[i] * __half2float(kn[i]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
            }
            const float mb = fmaxf(m, dot);
            const float corr = __expf(m - mb), p = __expf(dot - mb);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                acc[i] = acc[i] * corr + p * __half2float(vn[i]);
            }
            m = mb;
        }
        float* mine = parts + w.warp * (hd + 2);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            mine[w.lane * DPL + i] = acc[i];
        }
        if (w.lane == 0) {
            mine[hd] = m;
            mine[hd + 1] = l;
        }
        __syncthreads();
        if (threadIdx.x < hd) {
            const int e = threadIdx.x;
            float M = -INFINITY;
            for (int p = 0; p < MEGA_WARPS; ++p) {
                M = fmaxf(M, parts[p * (hd + 2) + hd]);
            }
            float s_acc = 0.0f, L = 0.0f;
            for (int p = 0; p < MEGA_WARPS; ++p) {
                const float mp = parts[p * (hd + 2) + hd];
                const float f = mp == -INFINITY ? 0.0f : __expf(mp - M);
                s_acc += parts[p * (hd + 2) + e] * f;
                L += parts[p * (hd + 2) + hd + 1] * f;
            }
            float* out = a.part + ((int64_t)head * a.nsplit + split) * (hd + 4);
            out[4 + e] = s_acc;
            if (e == 0) {
                out[0] = M;
                out[1] = L;
            }
        }
        __syncthreads();
        first = false;
    }
}

// ---- arg-max ------------------------------------------------------------------------------------

__device__ __forceinline__ void better(float& bv, int& bi, float v, int i)
{
    if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
    }
}

__device__ __forceinline__ void warp_best(float& bv, int& bi)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        better(bv, bi, ov, oi);
    }
}

// Greedy choice, lowest index on ties.  Each CTA scans its slice of the logits.
__device__ __noinline__ void argmax_slice(const MegaArgs& a, const float* logits, int warp, int lane, uint8_t* smem,
                                             const MegaSmem& sm)
{
    float* sv = reinterpret_cast<float*>(smem + sm.red);
    int* si = reinterpret_cast<int*>(smem + sm.red) + MEGA_WARPS;
    const int per = (a.vocab + gridDim.x - 1) / gridDim.x;
    const int i0 = blockIdx.x * per, i1 = min(a.vocab, i0 + per);
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = i0 + threadIdx.x; i < i1; i += MEGA_THREADS) {
        better(bv, bi, __ldcg(logits + i), i);
    }
    warp_best(bv, bi);
    if (lane == 0) {
        sv[warp] = bv;
        si[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int p = 1; p < MEGA_WARPS; ++p) {
            better(bv, bi, sv[p], si[p]);
        }
        a.cand[2 * blockIdx.x] = __float_as_int(bv);
        a.cand[2 * blockIdx.x + 1] = bi;
    }
}

__device__ __noinline__ void commit_token(const MegaArgs& a, int warp, int lane)
{
    if (blockIdx.x != 0 || warp != 0) {
        return;
    }
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int b = lane; b < (int)gridDim.x; b += 32) {
        better(bv, bi, __int_as_float(__ldcg(a.cand + 2 * b)), __ldcg(a.cand + 2 * b + 1));
    }
    warp_best(bv, bi);
    if (lane == 0) {
        *a.token = bi;
        a.out_tokens[*a.out_count] = bi;
        *a.out_count += 1;
        *a.pos += 1;
    }
}

// ---- the token ----------------------------------------------------------------------------------

// Linear k of block l (k = 0..3: qkv, attn_output, gate|up, down); block n_layers holds only the
// output head.  One loop body serves every linear so that the multiply code exists once.
template <int DPL>
__device__ __forceinline__ bool run_token(const MegaArgs& a, Warp& w, uint8_t* smem, const MegaSmem& sm, int pos,
                                          unsigned int& target)
{
    int* s_flag = reinterpret_cast<int*>(smem + sm.flag);
    const int L = a.n_layers;
    for (int s = 0; s <= 4 * L; ++s) {
        const int l = s >> 2, k = s & 3;
        const MegaLinear* lin = a.lin + s;
        const MegaLayer ly = a.layers[l < L ? l : L - 1];
        if (s == 0) {
            stage_embed(a, smem, sm);
        }
        if (k == 0) {
            stage_norm(a, s == 0 ? nullptr : lin[-1].y, l < L ? ly.attn_norm : a.final_norm, lin[0].kc, w.warp, w.lane,
                       smem, sm);
        } else if (k == 1) {
            stage_ctx(a, lin[0].kc, w.warp, w.lane, smem, sm);
        } else if (k == 2) {
            stage_norm(a, lin[-1].y, ly.ffn_norm, lin[0].kc, w.warp, w.lane, smem, sm);
        } else {
            stage_swiglu(a, lin[-1].y, lin[0].kc, w.warp, w.lane, smem, sm);
        }
        run_linear(a, s, w, smem, sm);
        if (k == 0 && l < L) {
            AttnPre<DPL> pre;
            attn_preload<DPL>(a, ly, pos, w, pre);
            if (!grid_barrier(a, target, s_flag, w.ok)) {
                return false;
            }
            attn_stage<DPL>(a, ly, lin[0].y, pos, w, pre, smem, sm);
        }
        if (!grid_barrier(a, target, s_flag, w.ok)) {
            return false;
        }
    }
    argmax_slice(a, a.lin[4 * L].y, w.warp, w.lane, smem, sm);
    if (!grid_barrier(a, target, s_flag, w.ok)) {
        return false;
    }
    commit_token(a, w.warp, w.lane);
    return true;
}

template <int DPL>  // head_dim / 32
__global__ void __launch_bounds__(MEGA_THREADS, 1) llama_mega_kernel(const __grid_constant__ MegaArgs a)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const MegaSmem sm(a.d_model, a.hd, a.kc_max, 4 * a.n_layers + 1);
    Warp w;
    w.warp = threadIdx.x >> 5;
    w.lane = threadIdx.x & 31;
    w.ok = true;
    w.ring.base = smem + sm.ring + w.warp * MEGA_RING_BYTES;
    w.ring.bars = reinterpret_cast<uint64_t*>(smem + sm.bars) + w.warp * MEGA_MAX_SLOTS;
    w.ring.tb = 0;
    w.ring.ns = 0;
    w.ring.qi = 0;
    w.ring.qc = 0;
    w.ring.phase = 0;
    w.ring.issued = 0;
    w.ring.consumed = 0;
    if (w.lane == 0) {
        for (int s = 0; s < MEGA_MAX_SLOTS; ++s) {
            mbar_init(w.ring.bars + s, 1);
        }
        fence_barrier_init();
    }
    if (threadIdx.x < 128) {
        reinterpret_cast<uint32_t*>(smem + sm.zeros)[threadIdx.x] = 0u;
    }
    __syncwarp();
    // start this warp's weight stream
    const int n_lin = 4 * a.n_layers + 1;
    // the table of linears is read at every tile refill: keep it in shared memory
    {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a.lin);
        uint32_t* dst = reinterpret_cast<uint32_t*>(smem + sm.table);
        const int words = n_lin * (int)(sizeof(MegaLinear) / 4);
        for (int i = threadIdx.x; i < words; i += MEGA_THREADS) {
            dst[i] = src[i];
        }
    }
    __syncthreads();
    const MegaLinear* lin_s = reinterpret_cast<const MegaLinear*>(smem + sm.table);
    w.pf.s = 0;
    cursor_enter(w.pf, lin_s, n_lin, w.warp);
    ring_fill(w.ring, w.pf, lin_s, n_lin, w.warp, w.lane);
    const int pos = *a.pos;
    unsigned int target = 0;
    __syncthreads();

    const bool done = run_token<DPL>(a, w, smem, sm, pos, target);

    if (!done) {
        // leave nothing in flight: wait (bounded) for the copies this warp still has outstanding
        while ((int)(w.ring.issued - w.ring.consumed) > 0) {
            mbar_wait(w.ring.bars + w.ring.qc, (w.ring.phase >> w.ring.qc) & 1u);
            w.ring.phase ^= 1u << w.ring.qc;
            w.ring.qc = w.ring.qc + 1 == w.ring.ns ? 0 : w.ring.qc + 1;
            ++w.ring.consumed;
        }
    }
    // the last CTA out re-arms the counters for the next launch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(a.sync + 1, 1u);
        if (old == gridDim.x - 1) {
            a.sync[0] = 0u;
            a.sync[1] = 0u;
            __threadfence();
        }
    }
}

}  // namespace

int ll_mega_pick_wpr(int rt, int kc, int grid)
{
    int best = MEGA_WARPS;
    long best_cost = -1;
    for (int wpr = 2; wpr <= MEGA_WARPS; ++wpr) {
        if (MEGA_WARPS % wpr != 0 || MEGA_WARPS / wpr > 14) {  // named barriers 1..15 serve the groups
            continue;
        }
        const long groups = (long)grid * (MEGA_WARPS / wpr);
        const long cost = ((rt + groups - 1) / groups) * ((kc + wpr - 1) / wpr);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = wpr;
        }
    }
    return best;
}

size_t ll_mega_smem_bytes(int d_model, int hd, int kc_max, int n_layers)
{
    return (size_t)MegaSmem(d_model, hd, kc_max, 4 * n_layers + 1).total;
}

cudaError_t ll_mega_decode(const MegaArgs& args, int grid, cudaStream_t st)
{
    const size_t smem = ll_mega_smem_bytes(args.d_model, args.hd, args.kc_max, args.n_layers);
    if (smem > 227 * 1024 || (args.hd != 64 && args.hd != 128)) {
        return cudaErrorInvalidConfiguration;
    }
    static size_t configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return e;
    }
    const void* kernel = args.hd == 64 ? reinterpret_cast<const void*>(llama_mega_kernel<2>)
                                       : reinterpret_cast<const void*>(llama_mega_kernel<4>);
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        for (const void* k : {reinterpret_cast<const void*>(llama_mega_kernel<2>),
                              reinterpret_cast<const void*>(llama_mega_kernel<4>)}) {
            e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) {
                return e;
            }
        }
        if (dev >= 0 && dev < 64) {
            configured[dev] = smem;
        }
    }
    MegaArgs a = args;
    void* params[] = {&a};
    return cudaLaunchCooperativeKernel(kernel, dim3((unsigned)grid), dim3(MEGA_THREADS), params, smem, st);
}

}  // namespace qmm

// Shared definitions of the packed ("repacked at upload") weight layout and of the
// packed activation layout used by the sm_100a kernels.
//
// A [N,K] GGUF tensor (N output rows, quant blocks running along K within a row,
// tools/gguf/GGUFImporter.cpp:206-221) is cut into tiles of 16 rows x 256 columns,
// stored tile after tile ([row tile][K chunk]) so that one tile is ONE contiguous,
// 16-byte-aligned run of bytes: a single TMA bulk copy (cp.async.bulk) brings it
// into shared memory, and the tiles of one row tile follow each other in memory.
// 16 rows is the M extent of one integer tensor-core MMA (mma.sync m16n8k32 /
// m16n8k16) with the weights as the A operand; 256 columns is one K-quant
// super-block = eight 32-wide blocks.  Inside a tile the quants and the scales are
// separate planes, and the quant plane is stored in the order the MMA A-fragment
// wants it, 16 bytes per lane, so a warp reads a fragment group as one
// conflict-free 512-byte access and needs no shuffles:
//
//   lane = 4*g + t   (g = lane>>2 selects rows g and g+8, t = lane&3 selects k-slots
//                     4t..4t+3 and 16+4t..16+4t+3 of a 32-wide block)
//
// Rows beyond N and blocks beyond K are padded with zero scales, so they add 0.
// A tile has exactly as many bytes as the 16 x 256 weights have in the ggml
// encoding (2304 / 4352 / 2304 / 3360), so HBM traffic equals the payload size.
//
// Planes of one tile, in storage order:
//   Q4_0  qs  [4 pairs][32 lanes][16 B]  words {blk 2p weights 4t.., blk 2p weights 16+4t..,
//                                         blk 2p+1 weights 4t.., blk 2p+1 weights 16+4t..};
//                                         byte i = weight +i of row g in the low nibble and
//                                         of row g+8 in the high nibble           2048 B
//         p1  [16 rows][8 blocks] fp16 d                                        256 B
//   Q8_0  qs  [8 blocks][32 lanes][16 B] {row g bytes 4t.., row g+8 bytes 4t..,
//                                         row g bytes 16+4t.., row g+8 bytes 16+4t..} 4096 B
//         p1  [16 rows][8 blocks] fp16 d                                        256 B
//   Q4_K  qs  [4 pairs][32 lanes][16 B]  as Q4_0 with sub-blocks 2p, 2p+1 of the super-block 2048 B
//         p1  [16 rows][12 B]            the 12 packed 6-bit scale/min bytes, as in ggml 192 B
//         p2  [16 rows] half2 (d, dmin)                                          64 B
//   Q6_K  qs  [6][32 lanes][16 B]        per lane 24 words, index ((quad*2+rsel)*3+j):
//                                         byte i of word j<3 holds in bits 7..2 the
//                                         6-bit quant (bit 5 flipped) of sub-block
//                                         4*quad+j, weight 4t+i, row g+8*rsel, and in
//                                         bits 1..0 a third of the quant of sub-block
//                                         4*quad+3 (j=0: bits 5..4, 1: 3..2, 2: 1..0)  3072 B
//         p1  [16 rows][16] int8 sub-block scales                               256 B
//         p2  [16 rows] fp16 d                                                   32 B
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qmm {

constexpr int FMT_Q4_0 = 1;
constexpr int FMT_Q8_0 = 5;
constexpr int FMT_Q4_K = 9;
constexpr int FMT_Q6_K = 11;
// Formats the importer carries as payloads and this library only dequantizes (no tile layout, no matmul).
constexpr int FMT_Q4_1 = 2;
constexpr int FMT_Q5_0 = 3;
constexpr int FMT_Q5_1 = 4;
constexpr int FMT_Q2_K = 7;
constexpr int FMT_Q3_K = 8;
constexpr int FMT_Q5_K = 10;

constexpr int TILE_ROWS = 16;
constexpr int TILE_K = 256;

__host__ __device__ constexpr int block_elems(int fmt)
{
    return (fmt == FMT_Q4_0 || fmt == FMT_Q8_0 || fmt == FMT_Q4_1 || fmt == FMT_Q5_0 || fmt == FMT_Q5_1)
               ? 32
               : ((fmt == FMT_Q4_K || fmt == FMT_Q6_K || fmt == FMT_Q2_K || fmt == FMT_Q3_K || fmt == FMT_Q5_K) ? 256 : 0);
}
__host__ __device__ constexpr int block_bytes(int fmt)
{
    return fmt == FMT_Q4_0   ? 18
           : fmt == FMT_Q8_0 ? 34
           : fmt == FMT_Q4_K ? 144
           : fmt == FMT_Q6_K ? 210
           : fmt == FMT_Q4_1 ? 20
           : fmt == FMT_Q5_0 ? 22
           : fmt == FMT_Q5_1 ? 24
           : fmt == FMT_Q2_K ? 84
           : fmt == FMT_Q3_K ? 110
           : fmt == FMT_Q5_K ? 176
                             : 0;
}
// bytes per tile of each plane
__host__ __device__ constexpr int tile_qs_bytes(int fmt)
{
    return fmt == FMT_Q4_0 ? 2048 : fmt == FMT_Q8_0 ? 4096 : fmt == FMT_Q4_K ? 2048 : fmt == FMT_Q6_K ? 3072 : 0;
}
__host__ __device__ constexpr int tile_p1_bytes(int fmt)
{
    return fmt == FMT_Q4_K ? 192 : 256;
}
__host__ __device__ constexpr int tile_p2_bytes(int fmt)
{
    return fmt == FMT_Q4_K ? 64 : fmt == FMT_Q6_K ? 32 : 0;
}

// bytes of one whole tile, and where its planes start
__host__ __device__ constexpr int tile_bytes(int fmt)
{
    return tile_qs_bytes(fmt) + tile_p1_bytes(fmt) + tile_p2_bytes(fmt);
}
__host__ __device__ constexpr int tile_p1_offset(int fmt)
{
    return tile_qs_bytes(fmt);
}
__host__ __device__ constexpr int tile_p2_offset(int fmt)
{
    return tile_qs_bytes(fmt) + tile_p1_bytes(fmt);
}

// Device view of a packed weight (passed to kernels by value).
struct WeightView {
    const uint8_t* tiles;  // [rt][kc] tiles of tile_bytes(fmt)
    int64_t n;   // real rows
    int64_t k;   // real columns
    int rt;      // row tiles  = ceil(n / 16)
    int kc;      // K chunks   = ceil(k / 256)
    int fmt;
};

// Packed activations for the integer-MMA GEMV.  x[m,k] is quantized per (row m, 32-wide block
// of k) to 16 bits, x ~= xs * (256*hi + lo) with hi and lo both signed bytes
// (|256*hi + lo| <= 32639, xs = max|x| of the block / 32639), and stored in B-fragment order.
// The 32-wide granule is the quantization block of every weight format, so one integer block
// sum meets exactly one weight scale and one activation scale, and an outlier activation costs
// precision only inside its own block.  One MMA covers a group of four activation rows: column
// 2r carries the high bytes and column 2r+1 the low bytes of row 4*j + r.
// The buffer is an array of per-chunk records (one 256-wide K chunk each), so whoever produces
// 32 consecutive activations can write their block without knowing the rest:
//   general (m > 1), ncp = ceil(m / 4) column groups; record of XPK_XQ(ncp) + 2048 bytes:
//     xq   [8 blocks][ncp][32 lanes] uint2 {k-slots 4t..4t+3, 16+4t..16+4t+3} of column g
//     meta [8 blocks][16 rows] int4 {8*Q, 128*Q, float bits of xs, 0}
//   compact (m == 1): only lanes 0..7 (columns 0 and 1) exist; record of 640 bytes:
//     xq   [8 blocks][8 lanes] uint2        (lane = 4*digit + t, digit 0 = high byte)
//     meta [8 blocks] int4 {8*Q, 128*Q, float bits of xs, 0}
// Q = sum of the block's 16-bit quants: it turns the unsigned nibbles back into (n - 8) exactly,
// in integers, and carries the "- dmin*m" term of Q4_K.
struct XPackView {
    const uint8_t* base;  // [kc] records
    int kc;
    int ncp;
};

constexpr int XPK1_REC = 640;        // compact record
constexpr int XPK1_META = 512;       // offset of its meta part

__host__ __device__ inline int xpack_ncp(int m)
{
    return m <= 1 ? 1 : (m + 3) / 4;
}
__host__ __device__ constexpr int xpack_xq_bytes(int ncp)
{
    return 8 * ncp * 32 * 8;
}
__host__ __device__ constexpr int xpack_rec_bytes(int ncp)
{
    return xpack_xq_bytes(ncp) + 8 * 16 * 16;
}
__host__ __device__ inline size_t xpack_bytes(int kc, int ncp)
{
    return (size_t)kc * xpack_rec_bytes(ncp);
}
__host__ __device__ inline size_t xpack1_bytes(int kc)
{
    return (size_t)kc * XPK1_REC;
}

// Tensor-parallel epilogue of a batch-1 matvec whose result is one addend of a sum over ranks
// (the K-split attn_output and ffn_down): besides y, every result is stored into this rank's
// slot of each peer's receive buffer (peer memory mapped into this process) as one 8-byte
// packet {value bits, exchange number}.  The packet is written by a single store, so a reader
// that sees the expected exchange number also sees the value: no fence, no separate flag, and
// the cost of the exchange is one NVLink store latency.  n_peers == 0 switches it off.
constexpr int QMM_MAX_PEERS = 7;
struct PeerScatter {
    uint2* dst[QMM_MAX_PEERS];  // [n] packets in peer memory
    int n_peers;
    const int* pos;             // exchange number = *pos * sites + site + 1 (never 0)
    int sites, site;
    // Receiving side, used by the residual form (EPI_RESID_PACK), which finishes the sum over the ranks in the
    // same kernel: after a CTA has stored its 32 partial sums to the peers it polls the peers' packets for the
    // same rows in this rank's receive buffer (bounded), adds the addends in rank order (every rank gets the
    // same bits) and goes on with residual, packing and sum of squares.  A CTA sends before it waits and waits
    // for other GPUs only, so ranks cannot block each other.
    const uint2* recv;          // [tp_size][n] packets {value bits, exchange number}; own slot unused
    int tp_rank, tp_size;
    unsigned int spin_limit;    // polls of one packet before giving up
    int* wait_status;           // set to 5 when a packet did not come; non-zero: nothing waits again
};

// What a batch-1 matvec does besides multiplying (qmm_gemv_kernel.cuh).
// Input side:
//   x_f32 != null    the activations are an fp32 vector [k] in global memory; every CTA packs them into
//                    its own shared memory itself (no separate packing kernel, no packed buffer)
//   ss_in != null    the producer packed the activations WITHOUT their RMSNorm factor and left one sum
//                    of squares per 32 activations; the row sums are multiplied by
//                    s_in = 1/sqrt(sum(ss_in[0..ss_count)) / d_in + eps)
// Output side (mode):
//   EPI_STORE        y[row] = sum * s_in
//   EPI_RESID_PACK   h_out[row] = h_in[row] + sum * s_in; the matvec that follows reads
//                    RMSNorm(h_out) * norm_w, so the epilogue writes h_out * norm_w as packed activations
//                    (packed_out) and the sum of squares of its 32 rows (ss_out[n / 32], doubles); the
//                    1/rms factor is a scalar and is applied by the consumer (ss_in above).  A CTA of
//                    this form owns two row tiles = one 32-wide quantization block of the output.
//   EPI_SWIGLU       rows are interleaved gate/up: tile rows 0..7 = gate channels 8*tile..8*tile+7, rows
//                    8..15 = the same channels of up; y[channel] = silu(gate * s_in) * (up * s_in)
//   EPI_SWIGLU_PACK  the same product written as the packed input of the matvec that follows (packed_out;
//                    y optional): a CTA of this form owns four row tiles = 32 channels = one quantization block
constexpr int EPI_STORE = 0;
constexpr int EPI_RESID_PACK = 1;
constexpr int EPI_SWIGLU = 2;
constexpr int EPI_SWIGLU_PACK = 3;
// Row tiles one CTA owns in each form.
__host__ __device__ constexpr int epi_tiles(int epi)
{
    return epi == EPI_RESID_PACK ? 2 : epi == EPI_SWIGLU_PACK ? 4 : 1;
}
struct GemvFuse {
    int mode;
    const float* x_f32;
    const double* ss_in;
    int ss_count;
    int d_in;
    float eps;
    const float* h_in;    // EPI_RESID_PACK; may equal h_out
    float* h_out;
    const float* norm_w;  // weights of the norm the consumer applies
    double* ss_out;       // [n / 32]
    uint8_t* packed_out;  // compact packed-activation records of the consumer's input
};

__device__ __forceinline__ float half_bits_to_float(uint16_t h)
{
    return __half2float(__ushort_as_half(h));
}

// Q4_K: the j-th (scale, min) pair of the 12 packed bytes.
__host__ __device__ inline void q4k_scale_min(int j, const uint8_t* s, uint8_t& sc, uint8_t& mn)
{
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// Q6_K: raw 6-bit quant (0..63) of element e (0..255) of a raw 210-byte super-block.
__host__ __device__ inline uint32_t q6k_raw_quant(const uint8_t* blk, int e)
{
    const int h = e >> 7;
    const int r = e & 127;
    const int grp = r >> 5;
    const int l = r & 31;
    const uint8_t qlb = blk[64 * h + l + ((grp & 1) ? 32 : 0)];
    const uint32_t low = (grp & 2) ? (uint32_t)(qlb >> 4) : (uint32_t)(qlb & 0x0F);
    const uint32_t high = ((uint32_t)blk[128 + 32 * h + l] >> (2 * grp)) & 3u;
    return low | (high << 4);
}

}  // namespace qmm

// Index arithmetic of the upload-time repack and of the bit-exact dequantizer,
// written as __host__ __device__ functions so the same code can be exercised by a
// host-compiled test as well as by the kernels in qmm_repack.cu / qmm_dequant.cu.
#pragma once

#include "qmm_common.cuh"

namespace qmm {

// Where a shard's data sits inside the raw ggml payload of the full tensor.
struct RawSource {
    const uint8_t* base;   // first byte of the full payload
    int64_t row_bytes;     // bytes of one full row of the raw tensor
    int64_t row0;          // first raw row of this shard
    int64_t blk0;          // first raw block (of this format's block size) within a row
    int64_t n;             // rows in the shard
    int64_t nblk;          // blocks per row in the shard
};

__host__ __device__ inline const uint8_t* raw_block(const RawSource& s, int fmt, int64_t row, int64_t blk)
{
    return s.base + (s.row0 + row) * s.row_bytes + (s.blk0 + blk) * block_bytes(fmt);
}

__host__ __device__ inline uint32_t load_u32_unaligned(const uint8_t* p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

__host__ __device__ inline uint16_t load_u16_unaligned(const uint8_t* p)
{
    return (uint16_t)((uint32_t)p[0] | ((uint32_t)p[1] << 8));
}

// Number of 32-bit words in one tile.
__host__ __device__ constexpr int tile_words(int fmt)
{
    return tile_bytes(fmt) / 4;
}

// 4-bit quant of weight e (0..31) of block `sb` as stored in a raw ggml block:
// Q4_0 (sb ignored): byte e&15, low nibble for e<16; Q4_K: sub-block sb of the super-block.
__host__ __device__ inline uint32_t raw_nibble(int fmt, const uint8_t* blk, int sb, int e)
{
    if (fmt == FMT_Q4_0) {
        const uint8_t byte = blk[2 + (e & 15)];
        return (e >> 4) ? (uint32_t)(byte >> 4) : (uint32_t)(byte & 15);
    }
    const uint8_t byte = blk[16 + 32 * (sb >> 1) + e];
    return (sb & 1) ? (uint32_t)(byte >> 4) : (uint32_t)(byte & 15);
}

// One 32-bit word of the packed qs plane.  `w` indexes the words of tile
// (tile_r, tile_c) in storage order: ((group * 32 + lane) * 4 + j).
__host__ __device__ inline uint32_t repack_qs_word(int fmt, const RawSource& s, int tile_r, int tile_c, int w)
{
    const int j = w & 3;
    const int lane = (w >> 2) & 31;
    const int grp = w >> 7;
    const int g = lane >> 2;
    const int t = lane & 3;
    if (fmt == FMT_Q4_0 || fmt == FMT_Q4_K) {
        // word j of pair `grp`: block (Q4_K: sub-block) 2*grp + (j>>1), weights 16*(j&1) + 4t + i;
        // byte i = row g in the low nibble, row g+8 in the high nibble
        const int sb = 2 * grp + (j >> 1);
        const int e0 = 16 * (j & 1) + 4 * t;
        uint32_t word = 0;
        for (int i = 0; i < 4; ++i) {
            uint32_t nib[2];
            for (int rs = 0; rs < 2; ++rs) {
                const int64_t row = (int64_t)tile_r * 16 + g + 8 * rs;
                const int64_t blk = fmt == FMT_Q4_0 ? (int64_t)tile_c * 8 + sb : (int64_t)tile_c;
                nib[rs] = (row < s.n && blk < s.nblk) ? raw_nibble(fmt, raw_block(s, fmt, row, blk), sb, e0 + i)
                                                       : (fmt == FMT_Q4_0 ? 8u : 0u);
            }
            word |= (nib[0] | (nib[1] << 4)) << (8 * i);
        }
        return word;
    }
    if (fmt == FMT_Q8_0) {
        const int64_t row = (int64_t)tile_r * 16 + g + 8 * (j & 1);
        const int64_t blk = (int64_t)tile_c * 8 + grp;
        if (row >= s.n || blk >= s.nblk) {
            return 0u;
        }
        return load_u32_unaligned(raw_block(s, fmt, row, blk) + 2 + 4 * t + 16 * (j >> 1));
    }
    // Q6_K
    {
        const int W = 4 * grp + j;  // 0..23
        const int quad = W / 6;
        const int rsel = (W / 3) & 1;
        const int jj = W % 3;
        const int64_t row = (int64_t)tile_r * 16 + g + 8 * rsel;
        if (row >= s.n || tile_c >= s.nblk) {
            return 0u;
        }
        const uint8_t* blk = raw_block(s, fmt, row, tile_c);
        uint32_t word = 0;
        for (int i = 0; i < 4; ++i) {
            const uint32_t um = q6k_raw_quant(blk, 16 * (4 * quad + jj) + 4 * t + i) ^ 32u;
            const uint32_t u3 = q6k_raw_quant(blk, 16 * (4 * quad + 3) + 4 * t + i) ^ 32u;
            const uint32_t byte = (um << 2) | ((u3 >> (4 - 2 * jj)) & 3u);
            word |= byte << (8 * i);
        }
        return word;
    }
}

// One 32-bit word of plane p1; `w` counts words from the start of the plane.
__host__ __device__ inline uint32_t repack_p1_word(int fmt, const RawSource& s, int tile_r, int tile_c, int w)
{
    if (fmt == FMT_Q4_K) {
        const int r = w / 3;  // 12 bytes per row
        const int q = w % 3;
        const int64_t row = (int64_t)tile_r * 16 + r;
        if (row >= s.n || tile_c >= s.nblk) {
            return 0u;
        }
        return load_u32_unaligned(raw_block(s, fmt, row, tile_c) + 4 + 4 * q);
    }
    const int r = w >> 2;   // 16 bytes per row
    const int q = w & 3;
    const int64_t row = (int64_t)tile_r * 16 + r;
    if (row >= s.n) {
        return 0u;
    }
    if (fmt == FMT_Q4_0 || fmt == FMT_Q8_0) {
        uint32_t out = 0;
        for (int h = 0; h < 2; ++h) {
            const int64_t blk = (int64_t)tile_c * 8 + 2 * q + h;
            if (blk < s.nblk) {
                out |= (uint32_t)load_u16_unaligned(raw_block(s, fmt, row, blk)) << (16 * h);
            }
        }
        return out;
    }
    if (tile_c >= s.nblk) {
        return 0u;
    }
    return load_u32_unaligned(raw_block(s, fmt, row, tile_c) + 192 + 4 * q);  // Q6_K int8 scales
}

// One 32-bit word of plane p2: Q4_K (d, dmin) of row w; Q6_K the fp16 d of rows 2w and 2w+1.
__host__ __device__ inline uint32_t repack_p2_word(int fmt, const RawSource& s, int tile_r, int tile_c, int w)
{
    if (tile_c >= s.nblk) {
        return 0u;
    }
    if (fmt == FMT_Q4_K) {
        const int64_t row = (int64_t)tile_r * 16 + w;
        return row < s.n ? load_u32_unaligned(raw_block(s, fmt, row, tile_c)) : 0u;
    }
    uint32_t out = 0;
    for (int h = 0; h < 2; ++h) {
        const int64_t row = (int64_t)tile_r * 16 + 2 * w + h;
        if (row < s.n) {
            out |= (uint32_t)load_u16_unaligned(raw_block(s, fmt, row, tile_c) + 208) << (16 * h);
        }
    }
    return out;
}

// One 32-bit word of a packed tile; `w` counts words from the start of the tile.
__host__ __device__ inline uint32_t repack_tile_word(int fmt, const RawSource& s, int tile_r, int tile_c, int w)
{
    const int qw = tile_qs_bytes(fmt) / 4;
    const int p1w = tile_p1_bytes(fmt) / 4;
    if (w < qw) {
        return repack_qs_word(fmt, s, tile_r, tile_c, w);
    }
    if (w < qw + p1w) {
        return repack_p1_word(fmt, s, tile_r, tile_c, w - qw);
    }
    return repack_p2_word(fmt, s, tile_r, tile_c, w - qw - p1w);
}

__host__ __device__ inline float fp16_bits_to_float(uint16_t h)
{
    return __half2float(__ushort_as_half(h));
}

// Multiplication / subtraction with one rounding each.  Device code must not let
// the compiler contract a*b-c into an FMA, or the result stops being bit-exact.
__host__ __device__ inline float mul_rn(float a, float b)
{
#ifdef __CUDA_ARCH__
    return __fmul_rn(a, b);
#else
    volatile float r = a * b;
    return r;
#endif
}
__host__ __device__ inline float sub_rn(float a, float b)
{
#ifdef __CUDA_ARCH__
    return __fsub_rn(a, b);
#else
    volatile float r = a - b;
    return r;
#endif
}
__host__ __device__ inline float add_rn(float a, float b)
{
#ifdef __CUDA_ARCH__
    return __fadd_rn(a, b);
#else
    volatile float r = a + b;
    return r;
#endif
}

// Value of element (row, col) of the packed weight; bit-exact with ggml's to_float.
__host__ __device__ inline float dequant_packed_element(const WeightView& v, int64_t row, int64_t col)
{
    const int64_t tile = (row >> 4) * v.kc + (col >> 8);
    const int r = (int)(row & 15);
    const int g = r & 7;
    const int rs = r >> 3;
    const int ck = (int)(col & 255);
    const uint8_t* tb = v.tiles + tile * tile_bytes(v.fmt);
    const uint32_t* qs = reinterpret_cast<const uint32_t*>(tb);
    const uint8_t* p1 = tb + tile_p1_offset(v.fmt) + r * (v.fmt == FMT_Q4_K ? 12 : 16);
    const uint8_t* p2 = tb + tile_p2_offset(v.fmt);
    if (v.fmt == FMT_Q4_0 || v.fmt == FMT_Q8_0) {
        const int b = ck >> 5;
        const int e = ck & 31;
        const int t = (e & 15) >> 2;
        const int bi = e & 3;
        const int half = e >> 4;
        const int lane = 4 * g + t;
        const float d = fp16_bits_to_float(load_u16_unaligned(p1 + 2 * b));
        if (v.fmt == FMT_Q4_0) {
            const uint32_t word = qs[((b >> 1) * 32 + lane) * 4 + 2 * (b & 1) + half];
            const int nib = (int)((word >> (8 * bi + 4 * rs)) & 15u);
            return mul_rn((float)(nib - 8), d);
        }
        const uint32_t word = qs[(b * 32 + lane) * 4 + rs + 2 * half];
        const int q = (int)(int8_t)((word >> (8 * bi)) & 0xFFu);
        return mul_rn((float)q, d);
    }
    if (v.fmt == FMT_Q4_K) {
        const int sb = ck >> 5;
        const int e = ck & 31;
        const int bi = e & 3;
        const int lane = 4 * g + ((e & 15) >> 2);
        const uint32_t word = qs[((sb >> 1) * 32 + lane) * 4 + 2 * (sb & 1) + (e >> 4)];
        const int nib = (int)((word >> (8 * bi + 4 * rs)) & 15u);
        const uint32_t dm = *reinterpret_cast<const uint32_t*>(p2 + r * 4);
        const float d = fp16_bits_to_float((uint16_t)(dm & 0xFFFFu));
        const float dmin = fp16_bits_to_float((uint16_t)(dm >> 16));
        uint8_t sc, mn;
        q4k_scale_min(sb, p1, sc, mn);
        const float d1 = mul_rn(d, (float)sc);
        const float m1 = mul_rn(dmin, (float)mn);
        return sub_rn(mul_rn(d1, (float)nib), m1);
    }
    // Q6_K
    {
        const int sb = ck >> 4;
        const int e = ck & 15;
        const int t = e >> 2;
        const int bi = e & 3;
        const int quad = sb >> 2;
        const int jj = sb & 3;
        const int lane = 4 * g + t;
        const int base = (quad * 2 + rs) * 3;
        uint32_t u;
        if (jj < 3) {
            const int W = base + jj;
            const uint32_t word = qs[((W >> 2) * 32 + lane) * 4 + (W & 3)];
            u = ((word >> (8 * bi)) & 0xFFu) >> 2;
        } else {
            u = 0;
            for (int j2 = 0; j2 < 3; ++j2) {
                const int W = base + j2;
                const uint32_t word = qs[((W >> 2) * 32 + lane) * 4 + (W & 3)];
                u |= ((word >> (8 * bi)) & 3u) << (4 - 2 * j2);
            }
        }
        const int q = (int)(u ^ 32u) - 32;
        const float d = fp16_bits_to_float(*reinterpret_cast<const uint16_t*>(p2 + r * 2));
        const float sc = (float)(int8_t)p1[sb];
        return mul_rn(mul_rn(d, sc), (float)q);
    }
}

// Value of element e of raw block `blk` (un-repacked ggml bytes).
__host__ __device__ inline float dequant_raw_element(int fmt, const uint8_t* blk, int e)
{
    if (fmt == FMT_Q4_0) {
        const float d = fp16_bits_to_float(load_u16_unaligned(blk));
        const uint8_t byte = blk[2 + (e & 15)];
        const int nib = (e >> 4) ? (byte >> 4) : (byte & 15);
        return mul_rn((float)(nib - 8), d);
    }
    if (fmt == FMT_Q8_0) {
        const float d = fp16_bits_to_float(load_u16_unaligned(blk));
        return mul_rn((float)(int8_t)blk[2 + e], d);
    }
    if (fmt == FMT_Q4_K) {
        const float d = fp16_bits_to_float(load_u16_unaligned(blk));
        const float dmin = fp16_bits_to_float(load_u16_unaligned(blk + 2));
        const int sb = e >> 5;
        uint8_t sc, mn;
        q4k_scale_min(sb, blk + 4, sc, mn);
        const uint8_t byte = blk[16 + 32 * (sb >> 1) + (e & 31)];
        const int nib = (sb & 1) ? (byte >> 4) : (byte & 15);
        return sub_rn(mul_rn(mul_rn(d, (float)sc), (float)nib), mul_rn(dmin, (float)mn));
    }
    if (fmt == FMT_Q6_K) {
        const float d = fp16_bits_to_float(load_u16_unaligned(blk + 208));
        const int q = (int)q6k_raw_quant(blk, e) - 32;
        const float sc = (float)(int8_t)blk[192 + (e >> 4)];
        return mul_rn(mul_rn(d, sc), (float)q);
    }
    // ---- formats that are only dequantized (published ggml block formats) ----
    if (fmt == FMT_Q4_1 || fmt == FMT_Q5_0 || fmt == FMT_Q5_1) {
        // fp16 d [, fp16 m] [, 32 high bits: bit e belongs to element e], 16 nibble bytes: element j = low nibble
        // of byte j, element 16 + j = high nibble
        const float d = fp16_bits_to_float(load_u16_unaligned(blk));
        const bool has_m = fmt != FMT_Q5_0, has_h = fmt != FMT_Q4_1;
        const int qh_off = has_m ? 4 : 2;
        const uint8_t* qs = blk + qh_off + (has_h ? 4 : 0);
        const uint8_t byte = qs[e & 15];
        int q = (e >> 4) ? (byte >> 4) : (byte & 15);
        if (has_h) {
            q |= ((blk[qh_off + (e >> 3)] >> (e & 7)) & 1) << 4;
        }
        if (!has_m) {
            return mul_rn((float)(q - 16), d);
        }
        return add_rn(mul_rn((float)q, d), fp16_bits_to_float(load_u16_unaligned(blk + 2)));
    }
    if (fmt == FMT_Q2_K) {
        // 16 bytes (low nibble scale, high nibble min per 16-wide sub-block), 64 bytes of 2-bit quants
        // (element 128h + 32j + p = bits 2j.. of qs[32h + p]), fp16 d, fp16 dmin
        const uint8_t sc = blk[e >> 4];
        const float d = fp16_bits_to_float(load_u16_unaligned(blk + 80));
        const float dmin = fp16_bits_to_float(load_u16_unaligned(blk + 82));
        const int q = (blk[16 + 32 * (e >> 7) + (e & 31)] >> (2 * ((e >> 5) & 3))) & 3;
        return sub_rn(mul_rn(mul_rn(d, (float)(sc & 15)), (float)q), mul_rn(dmin, (float)(sc >> 4)));
    }
    if (fmt == FMT_Q3_K) {
        // 32 bytes of high bits (bit e/32 of hmask[e%32]; clear = subtract 4), 64 bytes of 2-bit quants as in
        // Q2_K, 12 bytes with sixteen 6-bit scales (nibbles of bytes 0..7, bit pairs of bytes 8..11), fp16 d
        const int s = e >> 4;
        const uint8_t* sb = blk + 96;
        const int lo = s < 8 ? (sb[s] & 15) : (sb[s - 8] >> 4);
        const int hi = (sb[8 + (s & 3)] >> (2 * (s >> 2))) & 3;
        const float d = fp16_bits_to_float(load_u16_unaligned(blk + 108));
        const int ql = (blk[32 + 32 * (e >> 7) + (e & 31)] >> (2 * ((e >> 5) & 3))) & 3;
        const int hb = (blk[e & 31] >> (e >> 5)) & 1;
        return mul_rn(mul_rn(d, (float)((lo | (hi << 4)) - 32)), (float)(ql - (hb ? 0 : 4)));
    }
    // Q5_K: fp16 d, fp16 dmin, the 12 scale bytes of Q4_K, 32 bytes of high bits (bit e/32 of qh[e%32]), 128 nibble
    // bytes laid out as in Q4_K
    {
        const float d = fp16_bits_to_float(load_u16_unaligned(blk));
        const float dmin = fp16_bits_to_float(load_u16_unaligned(blk + 2));
        const int sub = e >> 5;
        uint8_t sc, mn;
        q4k_scale_min(sub, blk + 4, sc, mn);
        const uint8_t byte = blk[48 + 32 * (sub >> 1) + (e & 31)];
        const int q = ((sub & 1) ? (byte >> 4) : (byte & 15)) | (((blk[16 + (e & 31)] >> sub) & 1) << 4);
        return sub_rn(mul_rn(mul_rn(d, (float)sc), (float)q), mul_rn(dmin, (float)mn));
    }
}

}  // namespace qmm

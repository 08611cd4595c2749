/*
 * CPU oracle for the GGUF block-quantized matmul path (see qmm_oracle.h).
 * TEST INFRASTRUCTURE ONLY.  Build with -ffp-contract=off so that
 * `a*b - c` rounds twice, as the C reference does on a baseline x86-64 build.
 */
#include "qmm_oracle.h"

#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_block_elems(int fmt)
{
    switch (fmt) {
    case ORACLE_FMT_Q4_0: return 32;
    case ORACLE_FMT_Q8_0: return 32;
    case ORACLE_FMT_Q4_K: return 256;
    case ORACLE_FMT_Q6_K: return 256;
    case ORACLE_FMT_Q4_1: return 32;
    case ORACLE_FMT_Q5_0: return 32;
    case ORACLE_FMT_Q5_1: return 32;
    case ORACLE_FMT_Q2_K: return 256;
    case ORACLE_FMT_Q3_K: return 256;
    case ORACLE_FMT_Q5_K: return 256;
    default: return 0;
    }
}

int oracle_block_bytes(int fmt)
{
    switch (fmt) {
    case ORACLE_FMT_Q4_0: return 18;
    case ORACLE_FMT_Q8_0: return 34;
    case ORACLE_FMT_Q4_K: return 144;
    case ORACLE_FMT_Q6_K: return 210;
    case ORACLE_FMT_Q4_1: return 20;
    case ORACLE_FMT_Q5_0: return 22;
    case ORACLE_FMT_Q5_1: return 24;
    case ORACLE_FMT_Q2_K: return 84;
    case ORACLE_FMT_Q3_K: return 110;
    case ORACLE_FMT_Q5_K: return 176;
    default: return 0;
    }
}

/* ---- IEEE binary16 / bfloat16 helpers -------------------------------------------------- */

float oracle_fp16_to_fp32(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + (127 - 15)) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

uint16_t oracle_fp32_to_fp16(float f)
{
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or exactly 2^-25, ties to even -> 0) */
        return sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal result */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) {
        ++q; /* carries into the exponent field correctly */
    }
    return (uint16_t)(sign | (base + q));
}

uint16_t oracle_fp32_to_bf16(float f)
{
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) {
        return (uint16_t)((x >> 16) | 0x40u);
    }
    const uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

float oracle_bf16_to_fp32(uint16_t b)
{
    const uint32_t x = (uint32_t)b << 16;
    float f;
    memcpy(&f, &x, sizeof f);
    return f;
}

static inline uint16_t load_u16(const uint8_t* p)
{
    return (uint16_t)(p[0] | ((uint16_t)p[1] << 8));
}

/* ---- block dequantizers ------------------------------------------------------------------ */

/* Q8_0: fp16 d, then 32 int8 quants;  w = q * d. */
static void dequant_row_q8_0(const uint8_t* src, float* dst, int64_t k)
{
    const int64_t nb = k / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 34;
        const float d = oracle_fp16_to_fp32(load_u16(blk));
        const int8_t* q = (const int8_t*)(blk + 2);
        for (int j = 0; j < 32; ++j) {
            dst[b * 32 + j] = (float)q[j] * d;
        }
    }
}

/* Q4_0: fp16 d, then 16 bytes; byte j carries element j (low nibble) and
 * element 16+j (high nibble);  w = (nibble - 8) * d. */
static void dequant_row_q4_0(const uint8_t* src, float* dst, int64_t k)
{
    const int64_t nb = k / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 18;
        const float d = oracle_fp16_to_fp32(load_u16(blk));
        const uint8_t* qs = blk + 2;
        for (int j = 0; j < 16; ++j) {
            const int lo = (int)(qs[j] & 0x0F) - 8;
            const int hi = (int)(qs[j] >> 4) - 8;
            dst[b * 32 + j] = (float)lo * d;
            dst[b * 32 + 16 + j] = (float)hi * d;
        }
    }
}

/* The 12 scale bytes of a Q4_K super-block hold eight 6-bit scales and eight
 * 6-bit mins. */
static void q4k_scale_min(int j, const uint8_t* s, uint8_t* sc, uint8_t* mn)
{
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* Q4_K: fp16 d, fp16 dmin, 12 scale bytes, 128 nibble bytes.  Every 32-byte
 * group g of nibbles holds sub-block 2g in the low nibbles and 2g+1 in the
 * high nibbles;  w = (d*sc)*nibble - (dmin*m), each product rounded to fp32. */
static void dequant_row_q4_k(const uint8_t* src, float* dst, int64_t k)
{
    const int64_t nb = k / 256;
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 144;
        const float d = oracle_fp16_to_fp32(load_u16(blk));
        const float dmin = oracle_fp16_to_fp32(load_u16(blk + 2));
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        float* y = dst + b * 256;
        for (int g = 0; g < 4; ++g) {
            uint8_t sc, mn;
            q4k_scale_min(2 * g, scales, &sc, &mn);
            const float d1 = d * (float)sc;
            const float m1 = dmin * (float)mn;
            q4k_scale_min(2 * g + 1, scales, &sc, &mn);
            const float d2 = d * (float)sc;
            const float m2 = dmin * (float)mn;
            const uint8_t* q = qs + 32 * g;
            for (int l = 0; l < 32; ++l) {
                const float p1 = d1 * (float)(q[l] & 0x0F);
                const float p2 = d2 * (float)(q[l] >> 4);
                y[64 * g + l] = p1 - m1;
                y[64 * g + 32 + l] = p2 - m2;
            }
        }
    }
}

/* Q6_K: 128 bytes ql (low 4 bits), 64 bytes qh (high 2 bits), 16 int8 scales,
 * fp16 d.  Per 128-value half h and l in [0,32): values l, l+32, l+64, l+96 take
 * their low bits from ql[64h+l] lo, ql[64h+l+32] lo, ql[64h+l] hi, ql[64h+l+32] hi
 * and their high bits from bit pairs 0,2,4,6 of qh[32h+l]; q = 6-bit value - 32;
 * scale index 8h + l/16 + {0,2,4,6};  w = (d*scale)*q. */
static void dequant_row_q6_k(const uint8_t* src, float* dst, int64_t k)
{
    const int64_t nb = k / 256;
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * 210;
        const uint8_t* ql = blk;
        const uint8_t* qh = blk + 128;
        const int8_t* sc = (const int8_t*)(blk + 192);
        const float d = oracle_fp16_to_fp32(load_u16(blk + 208));
        float* y = dst + b * 256;
        for (int h = 0; h < 2; ++h) {
            for (int l = 0; l < 32; ++l) {
                const int is = 8 * h + l / 16;
                const uint8_t hb = qh[32 * h + l];
                const int q1 = (int)((ql[64 * h + l] & 0x0F) | (((hb >> 0) & 3) << 4)) - 32;
                const int q2 = (int)((ql[64 * h + l + 32] & 0x0F) | (((hb >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((ql[64 * h + l] >> 4) | (((hb >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((ql[64 * h + l + 32] >> 4) | (((hb >> 6) & 3) << 4)) - 32;
                const float s1 = d * (float)sc[is + 0];
                const float s2 = d * (float)sc[is + 2];
                const float s3 = d * (float)sc[is + 4];
                const float s4 = d * (float)sc[is + 6];
                y[128 * h + l] = s1 * (float)q1;
                y[128 * h + l + 32] = s2 * (float)q2;
                y[128 * h + l + 64] = s3 * (float)q3;
                y[128 * h + l + 96] = s4 * (float)q4;
            }
        }
    }
}

/* ---- formats that are only dequantized (published ggml block formats) ----------------------- */

static uint32_t load_u32(const uint8_t* p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

/* Q4_1: fp16 d, fp16 m, 16 nibble bytes (element j = low nibble of byte j, element 16+j = high nibble);
 * w = nibble*d + m, product and sum each rounded to fp32. */
static void dequant_row_q4_1(const uint8_t* src, float* dst, int64_t k)
{
    for (int64_t b = 0; b < k / 32; ++b) {
        const uint8_t* blk = src + b * 20;
        const float d = oracle_fp16_to_fp32(load_u16(blk));
        const float m = oracle_fp16_to_fp32(load_u16(blk + 2));
        const uint8_t* qs = blk + 4;
        for (int j = 0; j < 16; ++j) {
            const float p0 = (float)(qs[j] & 0x0F) * d;
            const float p1 = (float)(qs[j] >> 4) * d;
            dst[b * 32 + j] = p0 + m;
            dst[b * 32 + 16 + j] = p1 + m;
        }
    }
}

/* Q5_0: fp16 d, 32 high bits (bit e belongs to element e), 16 nibble bytes; w = (5-bit value - 16)*d. */
static void dequant_row_q5_0(const uint8_t* src, float* dst, int64_t k)
{
    for (int64_t b = 0; b < k / 32; ++b) {
        const uint8_t* blk = src + b * 22;
        const float d = oracle_fp16_to_fp32(load_u16(blk));
        const uint32_t qh = load_u32(blk + 2);
        const uint8_t* qs = blk + 6;
        for (int j = 0; j < 16; ++j) {
            const int q0 = (int)((qs[j] & 0x0F) | (((qh >> j) & 1u) << 4)) - 16;
            const int q1 = (int)((qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4)) - 16;
            dst[b * 32 + j] = (float)q0 * d;
            dst[b * 32 + 16 + j] = (float)q1 * d;
        }
    }
}

/* Q5_1: fp16 d, fp16 m, 32 high bits, 16 nibble bytes; w = (5-bit value)*d + m. */
static void dequant_row_q5_1(const uint8_t* src, float* dst, int64_t k)
{
    for (int64_t b = 0; b < k / 32; ++b) {
        const uint8_t* blk = src + b * 24;
        const float d = oracle_fp16_to_fp32(load_u16(blk));
        const float m = oracle_fp16_to_fp32(load_u16(blk + 2));
        const uint32_t qh = load_u32(blk + 4);
        const uint8_t* qs = blk + 8;
        for (int j = 0; j < 16; ++j) {
            const float p0 = (float)(int)((qs[j] & 0x0F) | (((qh >> j) & 1u) << 4)) * d;
            const float p1 = (float)(int)((qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4)) * d;
            dst[b * 32 + j] = p0 + m;
            dst[b * 32 + 16 + j] = p1 + m;
        }
    }
}

/* Q2_K: 16 bytes (low nibble = scale, high nibble = min of a 16-wide sub-block), 64 bytes of 2-bit quants,
 * fp16 d, fp16 dmin.  Element e = 128h + 32j + p (p < 32) is bits 2j..2j+1 of qs[32h + p]; its sub-block is
 * e / 16;  w = (d*scale)*q - (dmin*min). */
static void dequant_row_q2_k(const uint8_t* src, float* dst, int64_t k)
{
    for (int64_t b = 0; b < k / 256; ++b) {
        const uint8_t* blk = src + b * 84;
        const uint8_t* scales = blk;
        const uint8_t* qs = blk + 16;
        const float d = oracle_fp16_to_fp32(load_u16(blk + 80));
        const float dmin = oracle_fp16_to_fp32(load_u16(blk + 82));
        for (int e = 0; e < 256; ++e) {
            const int h = e >> 7, j = (e >> 5) & 3, p = e & 31;
            const uint8_t sc = scales[e >> 4];
            const float dl = d * (float)(sc & 0x0F);
            const float ml = dmin * (float)(sc >> 4);
            const float prod = dl * (float)((qs[32 * h + p] >> (2 * j)) & 3);
            dst[b * 256 + e] = prod - ml;
        }
    }
}

/* Q3_K: 32 bytes of high bits (bit e/32 of hmask[e%32]; a CLEAR bit subtracts 4), 64 bytes of 2-bit quants laid
 * out as in Q2_K, 12 bytes holding sixteen 6-bit scales (low 4 bits: nibbles of bytes 0..7, high 2 bits: bit
 * pairs of bytes 8..11), fp16 d;  w = (d*(scale - 32))*q with q in -4..3. */
static void dequant_row_q3_k(const uint8_t* src, float* dst, int64_t k)
{
    for (int64_t b = 0; b < k / 256; ++b) {
        const uint8_t* blk = src + b * 110;
        const uint8_t* hmask = blk;
        const uint8_t* qs = blk + 32;
        const uint8_t* sb = blk + 96;
        const float d = oracle_fp16_to_fp32(load_u16(blk + 108));
        for (int e = 0; e < 256; ++e) {
            const int s = e >> 4;
            const int lo = s < 8 ? (sb[s] & 0x0F) : (sb[s - 8] >> 4);
            const int hi = (sb[8 + (s & 3)] >> (2 * (s >> 2))) & 3;
            const float dl = d * (float)((lo | (hi << 4)) - 32);
            const int h = e >> 7, j = (e >> 5) & 3, p = e & 31;
            const int ql = (qs[32 * h + p] >> (2 * j)) & 3;
            const int hb = (hmask[p] >> (e >> 5)) & 1;
            dst[b * 256 + e] = dl * (float)(ql - (hb ? 0 : 4));
        }
    }
}

/* Q5_K: fp16 d, fp16 dmin, the 12 scale bytes of Q4_K, 32 bytes of high bits (bit e/32 of qh[e%32]), 128
 * nibble bytes as in Q4_K;  w = (d*sc)*(5-bit value) - (dmin*m). */
static void dequant_row_q5_k(const uint8_t* src, float* dst, int64_t k)
{
    for (int64_t b = 0; b < k / 256; ++b) {
        const uint8_t* blk = src + b * 176;
        const float d = oracle_fp16_to_fp32(load_u16(blk));
        const float dmin = oracle_fp16_to_fp32(load_u16(blk + 2));
        const uint8_t* scales = blk + 4;
        const uint8_t* qh = blk + 16;
        const uint8_t* qs = blk + 48;
        for (int e = 0; e < 256; ++e) {
            const int sub = e >> 5, p = e & 31;
            uint8_t sc, mn;
            q4k_scale_min(sub, scales, &sc, &mn);
            const float d1 = d * (float)sc;
            const float m1 = dmin * (float)mn;
            const uint8_t byte = qs[32 * (sub >> 1) + p];
            const int q = ((sub & 1) ? (byte >> 4) : (byte & 0x0F)) | (((qh[p] >> sub) & 1) << 4);
            const float prod = d1 * (float)q;
            dst[b * 256 + e] = prod - m1;
        }
    }
}

int oracle_dequant(int fmt, const uint8_t* payload, int64_t rows, int64_t k, float* out)
{
    const int elems = oracle_block_elems(fmt);
    const int bytes = oracle_block_bytes(fmt);
    if (elems == 0) {
        return -1;
    }
    if (k <= 0 || (k % elems) != 0) {
        return -2;
    }
    const int64_t row_bytes = (k / elems) * bytes;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t* src = payload + r * row_bytes;
        float* dst = out + r * k;
        switch (fmt) {
        case ORACLE_FMT_Q4_0: dequant_row_q4_0(src, dst, k); break;
        case ORACLE_FMT_Q8_0: dequant_row_q8_0(src, dst, k); break;
        case ORACLE_FMT_Q4_K: dequant_row_q4_k(src, dst, k); break;
        case ORACLE_FMT_Q4_1: dequant_row_q4_1(src, dst, k); break;
        case ORACLE_FMT_Q5_0: dequant_row_q5_0(src, dst, k); break;
        case ORACLE_FMT_Q5_1: dequant_row_q5_1(src, dst, k); break;
        case ORACLE_FMT_Q2_K: dequant_row_q2_k(src, dst, k); break;
        case ORACLE_FMT_Q3_K: dequant_row_q3_k(src, dst, k); break;
        case ORACLE_FMT_Q5_K: dequant_row_q5_k(src, dst, k); break;
        default: dequant_row_q6_k(src, dst, k); break;
        }
    }
    return 0;
}

/* ---- the fp32 matmul of the reference --------------------------------------------------- */

void oracle_transpose(const float* in, int64_t rows, int64_t cols, float* out)
{
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t c = 0; c < cols; ++c) {
            out[c * rows + r] = in[r * cols + c];
        }
    }
}

void oracle_matmul_ikj(const float* x, const float* wt, float* out, int64_t m, int64_t k, int64_t n)
{
    for (int64_t e = 0; e < m * n; ++e) {
        out[e] = 0.0f;
    }
    for (int64_t i = 0; i < m; ++i) {
        float* out_row = out + i * n;
        for (int64_t kk = 0; kk < k; ++kk) {
            const float lhs = x[i * k + kk];
            const float* rhs_row = wt + kk * n;
            for (int64_t j = 0; j < n; ++j) {
                out_row[j] += lhs * rhs_row[j];
            }
        }
    }
}

void oracle_matmul_ikj_mt(const float* x, const float* wt, float* out, int64_t m, int64_t k, int64_t n, int threads)
{
    if (threads < 1) {
        threads = 1;
    }
#pragma omp parallel num_threads(threads)
    {
#ifdef _OPENMP
        const int t = omp_get_thread_num();
        const int nt = omp_get_num_threads();
#else
        const int t = 0;
        const int nt = 1;
#endif
        const int64_t j0 = n * t / nt;
        const int64_t j1 = n * (t + 1) / nt;
        for (int64_t i = 0; i < m; ++i) {
            float* out_row = out + i * n;
            for (int64_t j = j0; j < j1; ++j) {
                out_row[j] = 0.0f;
            }
            for (int64_t kk = 0; kk < k; ++kk) {
                const float lhs = x[i * k + kk];
                const float* rhs_row = wt + kk * n;
                for (int64_t j = j0; j < j1; ++j) {
                    out_row[j] += lhs * rhs_row[j];
                }
            }
        }
    }
}

void oracle_matmul_nk(const float* x, const float* w, float* out, int64_t m, int64_t k, int64_t n, int threads)
{
    if (threads < 1) {
        threads = 1;
    }
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t j = 0; j < n; ++j) {
        const float* wr = w + j * k;
        for (int64_t i = 0; i < m; ++i) {
            const float* xr = x + i * k;
            float acc = 0.0f;
            for (int64_t kk = 0; kk < k; ++kk) {
                acc += xr[kk] * wr[kk];
            }
            out[i * n + j] = acc;
        }
    }
}

void oracle_matmul_nk_f64(const float* x, const float* w, double* out, int64_t m, int64_t k, int64_t n, int threads)
{
    if (threads < 1) {
        threads = 1;
    }
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t j = 0; j < n; ++j) {
        const float* wr = w + j * k;
        for (int64_t i = 0; i < m; ++i) {
            const float* xr = x + i * k;
            double acc = 0.0;
            for (int64_t kk = 0; kk < k; ++kk) {
                acc += (double)xr[kk] * (double)wr[kk];
            }
            out[i * n + j] = acc;
        }
    }
}

int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * CPU oracle for the GGUF block-quantized matmul path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA kernels and the timed CPU baseline, never a
 * product code path.
 *
 * What it restates (paths are relative to the LiteNN source tree):
 *   - tools/gguf/LLaMABuilder.cpp:66-162  row-wise block dequantization to fp32 [N,K]
 *     (the arithmetic itself is ggml's `to_float`, reached through
 *     ggml_get_type_traits(); ggml is an un-vendored git submodule
 *     third_party/llama.cpp whose pinned commit is not recorded, so the block
 *     formats are restated here from the published GGUF/ggml format description)
 *   - tools/gguf/LLaMABuilder.cpp:209-247  transpose [N,K] -> [K,N]
 *   - src/LiteNN/Device.h:628-660          fp32 i-k-j MatMul loop
 *
 * Parity pins: the 18-byte Q4_0 payload of tests/GGUFImporterTest.cpp:173-176
 * (values derived by hand from the format), and bit-exact agreement with the
 * `gguf` Python package's dequantizers on committed random fixtures.  The
 * reference's own tests hold no non-zero dequantized values or quantized matmul
 * outputs, so beyond those pins parity is "unpinned" by the reference itself.
 */
#ifndef QMM_ORACLE_H
#define QMM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Numeric values of LiteNN::QuantizedBlockFormat (src/LiteNN/Quantization.h:31-62). */
enum {
    ORACLE_FMT_Q4_0 = 1,
    ORACLE_FMT_Q8_0 = 5,
    ORACLE_FMT_Q4_K = 9,
    ORACLE_FMT_Q6_K = 11,
    /* formats the importer carries as payloads (tools/gguf/GGUFImporter.cpp:257-304) and the reference
     * dequantizes at lowering like the four above; here: dequantization only, no matmul kernels */
    ORACLE_FMT_Q4_1 = 2,
    ORACLE_FMT_Q5_0 = 3,
    ORACLE_FMT_Q5_1 = 4,
    ORACLE_FMT_Q2_K = 7,
    ORACLE_FMT_Q3_K = 8,
    ORACLE_FMT_Q5_K = 10,
};

/* elements / bytes per block (src/LiteNN/Quantization.h:186-217); 0 on unknown format. */
int oracle_block_elems(int fmt);
int oracle_block_bytes(int fmt);

float oracle_fp16_to_fp32(uint16_t h);
uint16_t oracle_fp32_to_fp16(float f);      /* round to nearest even */
uint16_t oracle_fp32_to_bf16(float f);      /* round to nearest even */
float oracle_bf16_to_fp32(uint16_t b);

/* Dequantize rows*k values laid out as rows of k/elems blocks.  Returns 0, or
 * -1 for an unknown format, -2 when k is not a multiple of the block size
 * (LLaMABuilder.cpp:121-126). */
int oracle_dequant(int fmt, const uint8_t* payload, int64_t rows, int64_t k, float* out);

/* [rows,cols] -> [cols,rows]  (Tensor::Transpose as used by MakeLinearFromArchive). */
void oracle_transpose(const float* in, int64_t rows, int64_t cols, float* out);

/* out[m,n] = sum_k x[m,k]*wt[k,n]; exactly the loop of Device.h:645-658:
 * zero-fill, then i / k / j with fp32 multiply and fp32 add (no FMA). */
void oracle_matmul_ikj(const float* x, const float* wt, float* out, int64_t m, int64_t k, int64_t n);

/* Same values as oracle_matmul_ikj but reads w as [N,K] (no transpose) and can
 * split the output rows over `threads` OpenMP threads: every out[i,j] is still
 * accumulated over k = 0..K-1 in order with separate multiply and add, so the
 * result is bit-identical to the reference loop. */
void oracle_matmul_nk(const float* x, const float* w, float* out, int64_t m, int64_t k, int64_t n, int threads);

/* Same reference loop, rows of `wt` columns split across threads (the labelled
 * "all host cores" baseline row). */
void oracle_matmul_ikj_mt(const float* x, const float* wt, float* out, int64_t m, int64_t k, int64_t n, int threads);

/* Double-accumulated dot products, used only to judge which of two fp32 results is closer. */
void oracle_matmul_nk_f64(const float* x, const float* w, double* out, int64_t m, int64_t k, int64_t n, int threads);

int oracle_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif

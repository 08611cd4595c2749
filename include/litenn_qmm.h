/*
 * litenn_qmm.h — C ABI of the B200 (sm_100a) block-quantized matmul path for LiteNN.
 *
 * The library keeps GGUF block-quantized weights (Q4_0, Q8_0, Q4_K, Q6_K) quantized
 * in HBM, repacked at upload time into tensor-core-fragment-ordered tiles, and
 * multiplies them with activations on the GPU.  It replaces, for this one path,
 * what LiteNN does today: dequantize every block tensor to fp32 on the host
 * (tools/gguf/LLaMABuilder.cpp:66-162), transpose it (LLaMABuilder.cpp:209-247) and
 * run the plain fp32 MatMul (src/LiteNN/Device.h:628-660 on the CPU device,
 * cublasSgemm in src/LiteNN/Device/CUDA.cpp:1344-1352 on the CUDA device).
 *
 * Conventions
 *   - Every function returns 0 on success or a negative QMM_E_* code; the message of
 *     the last failure on the calling thread is qmm_last_error().  LiteNN reports
 *     errors as std::runtime_error (src/LiteNN/Device/CUDA.cpp:89-131); the C++
 *     adapter in litenn_b200/host turns a non-zero status into that exception.
 *   - `fmt` takes the numeric values of LiteNN::QuantizedBlockFormat
 *     (src/LiteNN/Quantization.h:31-62).
 *   - `stream` is a cudaStream_t passed as void*, NULL = the default stream, as in
 *     LiteNN::CUDAExecutionOptions (src/LiteNN/Device/CUDA.h:70-74).  Calls only
 *     enqueue work; the caller synchronizes (the adapter honours `synchronize`).
 *   - Pointers named *_dev are device pointers on the weight's device, dense
 *     row-major, no strides — the same contract as DeviceTraits<CUDA>::DoBinaryOp
 *     (src/LiteNN/Device/CUDA.h:150-154).
 *   - There is no CPU fallback: without a usable CUDA device every compute entry
 *     point fails with QMM_E_CUDA.
 */
#ifndef LITENN_QMM_H
#define LITENN_QMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QMM_ABI_VERSION 2

/* LiteNN::QuantizedBlockFormat values (src/LiteNN/Quantization.h:31-62). */
#define QMM_FMT_Q4_0 1
#define QMM_FMT_Q8_0 5
#define QMM_FMT_Q4_K 9
#define QMM_FMT_Q6_K 11
/* Block formats the importer also carries as payloads (tools/gguf/GGUFImporter.cpp:257-304) and the
 * reference dequantizes at lowering through ggml's to_float like the four above.  This library knows
 * their layout (qmm_block_layout) and dequantizes them on the device (qmm_dequantize_raw), bit-exact;
 * it has no matmul kernels for them: qmm_weight_create refuses them. */
#define QMM_FMT_Q4_1 2
#define QMM_FMT_Q5_0 3
#define QMM_FMT_Q5_1 4
#define QMM_FMT_Q2_K 7
#define QMM_FMT_Q3_K 8
#define QMM_FMT_Q5_K 10

#define QMM_OK 0
#define QMM_E_INVALID (-1)     /* bad argument (shape, format, null pointer, batch too large) */
#define QMM_E_CUDA (-2)        /* a CUDA runtime call failed */
#define QMM_E_UNSUPPORTED (-3) /* valid request the library does not implement */
#define QMM_E_KERNEL (-4)      /* a kernel reported an error status */

/* Largest activation batch the GEMV entry points accept. */
#define QMM_GEMV_MAX_BATCH 16

/* How qmm_weight_create_shard cuts a [N,K] weight for tensor parallelism. */
#define QMM_SPLIT_NONE 0
#define QMM_SPLIT_N 1 /* contiguous output rows; no exchange afterwards */
#define QMM_SPLIT_K 2 /* block-aligned slice of every row; partial sums need an all-reduce */

/* Output element type of qmm_gemm_bf16. */
#define QMM_OUT_F32 0
#define QMM_OUT_BF16 1

typedef struct qmm_weight qmm_weight; /* opaque, device-resident packed weight */

typedef struct qmm_weight_info {
    int32_t fmt;
    int32_t device;
    int64_t n;            /* output features (rows of the GGUF tensor) held by this handle */
    int64_t k;            /* input features (row width) held by this handle */
    int64_t payload_bytes; /* bytes of the ggml payload this handle represents */
    int64_t packed_bytes;  /* bytes resident in HBM after the repack (incl. padding) */
} qmm_weight_info;

int qmm_abi_version(void);

/* Thread-local message of the last failing call ("" if none). */
const char* qmm_last_error(void);

/* Elements and bytes per block; replaces GetQuantizedBlockLayout
 * (src/LiteNN/Quantization.h:186-217) for the four supported formats. */
int qmm_block_layout(int fmt, int* elems_per_block, int* bytes_per_block);

/* Number of CUDA devices visible (0 when there is no driver or GPU). */
int qmm_device_count(void);

/*
 * Upload-time repack.  `payload` is the raw ggml block payload of a [n,k] tensor
 * exactly as the importer keeps it (Tensor<CPU>{UInt8,[nbytes]},
 * tools/gguf/GGUFImporter.cpp:478-491): n rows of k/elems blocks.  It may live on
 * the host (payload_on_device = 0) or already on `device`.  The validation mirrors
 * DequantizeGGMLVariable: k must be a multiple of the block size
 * (LLaMABuilder.cpp:121-126) and payload_bytes must equal rows * row_bytes
 * (LLaMABuilder.cpp:137-142).  The call synchronizes `stream` before returning so
 * the source buffer may be released.
 */
int qmm_weight_create(int device, int fmt, const void* payload, size_t payload_bytes, int payload_on_device,
                      int64_t n, int64_t k, void* stream, qmm_weight** out);

/*
 * Same, but keeps only this rank's shard: QMM_SPLIT_N takes rows
 * [rank*n/tp, (rank+1)*n/tp), QMM_SPLIT_K takes columns [rank*k/tp, (rank+1)*k/tp)
 * of every row.  n (resp. k) must divide evenly and a K shard must be a whole
 * number of blocks, else QMM_E_INVALID (never truncated).  `payload` is the FULL
 * tensor.  No counterpart in LiteNN, which has no tensor parallelism.
 */
int qmm_weight_create_shard(int device, int fmt, const void* payload, size_t payload_bytes, int payload_on_device,
                            int64_t n, int64_t k, int split, int tp_rank, int tp_size, void* stream,
                            qmm_weight** out);

int qmm_weight_destroy(qmm_weight* w);
int qmm_weight_get_info(const qmm_weight* w, qmm_weight_info* info);

/*
 * Dequantize the packed weight to fp32 [n,k] on the device.  Values are bit-exact
 * with ggml's to_float as called by DequantizeGGMLVariable (LLaMABuilder.cpp:147-150).
 * Verification aid; the matmul entry points never materialise this tensor.
 */
int qmm_dequantize(const qmm_weight* w, float* out_dev, void* stream);

/* Dequantize a raw (not repacked) ggml payload that already sits on the device: any of the ten
 * formats above.  Used to prove dequant(repacked) == dequant(raw), and as the device-side
 * replacement of DequantizeGGMLVariable (LLaMABuilder.cpp:66-162) for tensors in a format
 * without matmul kernels. */
int qmm_dequantize_raw(int device, int fmt, const void* payload_dev, int64_t n, int64_t k, float* out_dev,
                       void* stream);

/*
 * y[m,n] = x[m,k] · Wᵀ for a decode-sized batch, 1 <= m <= QMM_GEMV_MAX_BATCH,
 * fp32 activations and outputs, fp32 accumulation across blocks.  This is the
 * fused form of the graph pattern QuantizedConstant/VariableRef(UInt8 payload) ->
 * DequantizeNode{Block,[n,k],Float32} -> Transpose -> MatMul(x, ·)
 * (src/LiteNN/Graph.h:66-70,115-120; Layer/Linear.h:64-90) and stands where
 * DeviceTraits<CUDA>::DoBinaryOp(MatMul) (src/LiteNN/Device/CUDA.cpp:1914-1940)
 * is called today.  A packing kernel quantizes the activations first; its scratch memory
 * (the packed activations) comes from a per-(device,stream) workspace the library allocates
 * on first use.
 */
int qmm_gemv_f32(const qmm_weight* w, const float* x_dev, float* y_dev, int m, void* stream);

/*
 * The two halves of qmm_gemv_f32, for callers that multiply ONE activation with
 * several weights (q/k/v and gate/up in LLaMABuilder.cpp:502-557 all read the same
 * normalized hidden state): quantize and pack the activations once, then run any
 * number of matvecs on the packed form.  `packed_dev` is caller-owned device memory
 * of qmm_packed_activation_bytes(k, m) bytes, 16-byte aligned.  The packed form
 * depends on k and m only, not on the weight or its format: 16 bits per activation,
 * one scale per 32 consecutive activations (|error| <= 2^-16 of the block's largest
 * magnitude), stored in tensor-core fragment order.
 */
int qmm_packed_activation_bytes(int64_t k, int m, size_t* bytes);
int qmm_pack_activations(int device, const float* x_dev, int m, int64_t k, void* packed_dev, void* stream);
int qmm_gemv_packed(const qmm_weight* w, const void* packed_dev, float* y_dev, int m, void* stream);
/* Batch-1 packed activations back to fp32 [k] (the values the matvec actually multiplies). */
int qmm_unpack_activations(int device, const void* packed_dev, int64_t k, float* x_dev, void* stream);

/*
 * Fused batch-1 forms: a chain of matvecs without glue kernels in between.  They cover the
 * decoder-block pattern of LLaMABuilder.cpp:502-557 / :568-668 —
 *   x -> RMSNorm -> Linear -> ... -> Linear -> (+ residual) -> RMSNorm -> gate/up Linear ->
 *   SiLU(gate) * up (Layer/SwiGLU.h:54-64) -> down Linear -> (+ residual)
 * — by writing each matvec's result directly as the packed input of the next one.  RMSNorm
 * (ComputePrimitives.h:795-821, statistics in double) is split: RMSNorm(h) * w = (h * w) / rms(h).
 * The producer packs h * w and leaves one sum of squares per 32 elements of h (doubles); the
 * consumer multiplies ITS row sums by 1 / sqrt(sum / d_in + eps).
 *
 *   qmm_gemv_packed_rms       y = (x_packed . W^T) / rms, rms from ss_dev[0..ss_count)
 *   qmm_gemv_packed_residual  h += x_packed . W^T (in place, fp32 [n]); packed_out = pack(h * norm_w),
 *                             ss_out[n/32] = sums of squares of h; n must be a multiple of 32
 *   qmm_gemv_f32_residual     the same with fp32 activations x_dev [k], which the kernel packs itself
 *   qmm_gemv_packed_swiglu    W holds gate and up rows interleaved in groups of 8 (qmm_interleave_gate_up);
 *                             act_dev[n/2] = silu(gate . x / rms) * (up . x / rms), fp32; ss_dev may be
 *                             NULL (no 1/rms factor); n must be a multiple of 16
 *   qmm_gemv_packed_swiglu_pack  the same product written as the packed input of the down projection:
 *                             packed_out = pack(act) (qmm_packed_activation_bytes(n/2, 1) bytes, zeroed once by
 *                             the caller: blocks past n/2 are never written); act_dev may be NULL; n must be
 *                             a multiple of 64
 */
int qmm_gemv_packed_rms(const qmm_weight* w, const void* packed_dev, const double* ss_dev, int ss_count, int64_t d_in,
                        float eps, float* y_dev, void* stream);
int qmm_gemv_packed_residual(const qmm_weight* w, const void* packed_dev, float* h_dev, const float* norm_w_dev,
                             void* packed_out_dev, double* ss_out_dev, void* stream);
int qmm_gemv_f32_residual(const qmm_weight* w, const float* x_dev, float* h_dev, const float* norm_w_dev,
                          void* packed_out_dev, double* ss_out_dev, void* stream);
int qmm_gemv_packed_swiglu_pack(const qmm_weight* w_gate_up, const void* packed_dev, const double* ss_dev, int ss_count,
                                int64_t d_in, float eps, void* packed_out_dev, float* act_dev, void* stream);
int qmm_gemv_packed_swiglu(const qmm_weight* w_gate_up, const void* packed_dev, const double* ss_dev, int ss_count,
                           int64_t d_in, float eps, float* act_dev, void* stream);
/* Host helper: raw ggml payloads of ffn_gate and ffn_up ([n_each, k] each, n_each a multiple of 8)
 * into one [2*n_each, k] payload whose rows alternate 8 of gate, the same 8 of up. */
int qmm_interleave_gate_up(int fmt, const void* gate_host, const void* up_host, int64_t n_each, int64_t k, void* out_host);

/*
 * qmm_gemv_f32 for callers that must not allocate device memory while they run.
 * (No counterpart in LiteNN.)  Who needs it: a host thread that is inside a region
 * where cudaMalloc is forbidden or would stall everything — a latency-critical
 * serving loop that may not take the allocator's device-wide synchronization, a
 * process that has handed all free HBM to its KV cache, or code that replays work
 * under rules that exclude allocation.  qmm_gemv_f32 keeps the packed activations
 * in a workspace it cudaMallocs on first use per (device, stream); this variant keeps
 * them in a fixed array that is part of the library image instead, so it calls no
 * cudaMalloc, cudaFree or other allocating routine, ever.
 *
 * Limits and rules:
 *   - the packed activations must fit QMM_STATIC_SCRATCH_BYTES (640 KiB: k <= 16384 at
 *     m = 16, k <= 65536 at m = 4; at m = 1 the kernel's shared-memory plan binds first, as
 *     it does for qmm_gemv_f32); larger requests fail with QMM_E_INVALID;
 *   - the array exists once per GPU that loads the library and is held until the
 *     process exits; every call on that GPU shares it and finds the previous call's
 *     contents in it (each call rewrites all it reads), so two calls whose kernels
 *     may overlap on the GPU — different streams without ordering — race;
 *   - the first call on a device looks up the array's device address; make that call
 *     before starting any stream capture.
 */
#define QMM_STATIC_SCRATCH_BYTES (640 * 1024)
int qmm_gemv_f32_static(const qmm_weight* w, const float* x_dev, float* y_dev, int m, void* stream);

/*
 * y[m,n] = x[m,k] · Wᵀ for prefill: bf16 activations, weights dequantized tile by
 * tile to bf16 in shared memory and multiplied on the tcgen05 tensor cores with
 * fp32 accumulation in tensor memory.  out_dtype is QMM_OUT_F32 or QMM_OUT_BF16.
 */
int qmm_gemm_bf16(const qmm_weight* w, const void* x_bf16_dev, void* y_dev, int64_t m, int out_dtype,
                  void* stream);

/*
 * The same GEMM for fp32 callers: LiteNN's prefill graph is fp32 end to end and its MatMul takes any
 * number of rows (src/LiteNN/Device/CUDA.cpp:1344-1352; Layer/Linear.h:75-78).  The activations are
 * rounded to bf16 on the device (round to nearest even, into a per-(device, stream) workspace the
 * library allocates on first use), multiplied as above, and the result is fp32.  Against the
 * reference's fp32 product this adds the two bf16 roundings (activations and dequantized weights,
 * 2^-9 relative each); use qmm_gemv_f32 where m <= QMM_GEMV_MAX_BATCH and that matters.
 */
int qmm_gemm_f32(const qmm_weight* w, const float* x_dev, float* y_dev, int64_t m, void* stream);

/*
 * Host-buffer convenience used for end-to-end timing: copies x (host, fp32 [m,k])
 * to the device, runs qmm_gemv_f32, copies y back and synchronizes the stream —
 * the life of one MatMul node under Interpreter<CUDA> (src/LiteNN/Runtime/
 * Interpreter.h:343-354) with the weight already resident.
 */
int qmm_gemv_f32_host(const qmm_weight* w, const float* x_host, float* y_host, int m, void* stream);

/*
 * Every wait inside a kernel (on a copy landing in shared memory, on tensor-core
 * completion) has an iteration limit.  A kernel that ran out of it sets a per-device
 * status word and returns without finishing its output.  This call synchronizes
 * with the device, copies the word to *status_out, clears it, and returns
 * QMM_E_KERNEL if it was non-zero.  LiteNN has no counterpart: its CUDA backend
 * only wraps library calls (src/LiteNN/Device/CUDA.cpp:89-131).
 */
int qmm_kernel_status(int device, int* status_out);

/* cudaStreamSynchronize on `device`, for callers that do not link the CUDA runtime
 * themselves (the adapter's `synchronize = true`, src/LiteNN/Device/CUDA.cpp:1392-1395). */
int qmm_stream_synchronize(int device, void* stream);

/* Release every cached per-(device,stream) workspace. */
int qmm_release_workspaces(void);

#ifdef __cplusplus
}
#endif
#endif /* LITENN_QMM_H */

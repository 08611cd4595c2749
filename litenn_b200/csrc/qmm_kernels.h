// Host-callable launchers of the CUDA kernels (internal to the library).
#pragma once

#include "qmm_layout.cuh"

namespace qmm {

cudaError_t launch_repack(int fmt, const RawSource& src, int rt, int kc, uint8_t* tiles, int sm_count,
                          cudaStream_t stream);
cudaError_t launch_dequant_packed(const WeightView& v, float* out, int sm_count, cudaStream_t stream);
cudaError_t launch_dequant_raw(int fmt, const uint8_t* payload, int64_t n, int64_t k, float* out, int sm_count,
                               cudaStream_t stream);

// Quantize and pack x[m,k] (fp32) for the integer-MMA GEMV into `out`
// (xpack1_bytes(kc) bytes for m == 1, else xpack_bytes(kc, xpack_ncp(m))).
cudaError_t launch_pack_x(const float* x, int m, int64_t k, int kc, uint8_t* out, cudaStream_t stream);
// Compact (m == 1) packed activations back to fp32 [k]; verification aid.
cudaError_t launch_unpack_x(const uint8_t* packed, int64_t k, float* x, cudaStream_t stream);

// y[m,n] = x · Wᵀ from a packed weight and packed activations (launch_pack_x first).
// `status` points at a device int that a kernel sets non-zero if a bounded wait ran out.
cudaError_t launch_gemv(const WeightView& w, const XPackView& xp, float* y, int m, int* status, cudaStream_t stream);
// Batch 1 only when ps.n_peers > 0 (also scatters the result to the peers, PeerScatter) or when
// `fu` asks for an input RMSNorm factor or a fused epilogue (GemvFuse); both in qmm_common.cuh.
cudaError_t launch_gemv_fused(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                              const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream);
// per-format instantiations (qmm_gemv_<format>.cu)
cudaError_t launch_gemv_q4_0(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                             const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream);
cudaError_t launch_gemv_q8_0(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                             const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream);
cudaError_t launch_gemv_q4_k(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                             const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream);
cudaError_t launch_gemv_q6_k(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                             const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream);

// fp32 -> bf16, round to nearest even.
cudaError_t launch_f32_to_bf16(const float* x, int64_t count, void* out_bf16, cudaStream_t stream);

// Prefill GEMM on tcgen05: y[m,n] = x_bf16[m,k] · Wᵀ, fp32 or bf16 output.  On a
// configuration error `*why` explains it.
cudaError_t launch_gemm_bf16(const WeightView& w, const void* x_bf16, void* y, int64_t m, int out_bf16, int sm_count,
                             int* status, cudaStream_t stream, const char** why);

}  // namespace qmm

// Host-callable launchers of the CUDA kernels (internal to the library).
#pragma once

#include "qmm_layout.cuh"

namespace qmm {

cudaError_t launch_repack(int fmt, const RawSource& src, int rt, int kc, uint8_t* tiles, int sm_count,
                          cudaStream_t stream);
cudaError_t launch_dequant_packed(const WeightView& v, float* out, int sm_count, cudaStream_t stream);
cudaError_t launch_dequant_raw(int fmt, const uint8_t* payload, int64_t n, int64_t k, float* out, int sm_count,
                               cudaStream_t stream);

// Writable view of the packed activations (see XPackView).
struct XPackBuffers {
    uint4* xq;
    float* xs;
    float* xsum;
};

// Quantize and pack x[m,k] (fp32) for the integer-MMA GEMV.
cudaError_t launch_pack_x(const float* x, int m, int64_t k, int kc, int cg, const XPackBuffers& out,
                          cudaStream_t stream);

// y[m,n] = x · Wᵀ from a packed weight.  m == 1 reads the fp32 activations `x`
// directly; 2 <= m <= 16 reads the packed activations `xp` (launch_pack_x first).
// `status` points at a device int that a kernel sets non-zero if a bounded wait ran out.
cudaError_t launch_gemv(const WeightView& w, const float* x, const XPackView& xp, float* y, int m, int* status,
                        cudaStream_t stream);

}  // namespace qmm

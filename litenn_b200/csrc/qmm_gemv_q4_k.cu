// The Q4_K instantiations of the matvec kernel template (qmm_gemv_kernel.cuh).
#include "qmm_gemv_kernel.cuh"

namespace qmm {

cudaError_t launch_gemv_q4_k(const WeightView& w, const XPackView& xp, float* y, int m, int* status,
                           const PeerScatter& ps, const GemvFuse& fu, cudaStream_t stream)
{
    return launch_gemv_fmt<FMT_Q4_K>(w, xp, y, m, status, ps, fu, stream);
}

}  // namespace qmm

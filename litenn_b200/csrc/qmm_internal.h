// Declarations shared by the translation units behind the C ABI (qmm_api.cu, llama_decoder.cu).
#pragma once

#include <cuda_runtime.h>

#include "../../include/litenn_qmm.h"
#include "qmm_common.cuh"

// Records `message` as the calling thread's last error and returns `code`.
int qmm_internal_fail(int code, const char* message);
// The device's status word (what qmm_kernel_status reads), allocated on first use.
int qmm_internal_status_word(int device, int** out);
// The device-side view of a packed weight.
int qmm_internal_weight_view(const qmm_weight* w, qmm::WeightView* out);
// Batch-1 matvec on packed activations with an optional tensor-parallel scatter and an optional
// fused prologue/epilogue (qmm_common.cuh); `y_dev` may be null when the epilogue replaces it.
int qmm_internal_gemv_fused(const qmm_weight* w, const void* packed_dev, float* y_dev, const qmm::PeerScatter* scatter,
                            const qmm::GemvFuse* fuse, void* stream);

namespace qmm {

// Restores the caller's current device on scope exit, like LiteNN's CUDADeviceGuard
// (src/LiteNN/Device/CUDA.cpp:734-761).
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    cudaError_t err = cudaSuccess;
    explicit DeviceGuard(int device)
    {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) {
            err = cudaSetDevice(device);
        }
        ok = err == cudaSuccess;
    }
    ~DeviceGuard()
    {
        int now = -1;
        if (prev >= 0 && cudaGetDevice(&now) == cudaSuccess && now != prev) {
            cudaSetDevice(prev);
        }
    }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};

}  // namespace qmm

// Upload-time repack of raw ggml block payloads into the fragment-ordered planes
// described in qmm_common.cuh, and the bit-exact dequantizers used for verification.
// All kernels are plain gather/scatter over words; they run once per tensor at
// import time (the GPU-side replacement of the host loop in
// tools/gguf/LLaMABuilder.cpp:147-150), so they are written for clarity, with
// grid-stride loops sized to the device.
#include "qmm_kernels.h"
#include "qmm_layout.cuh"

namespace qmm {

namespace {

__global__ void repack_kernel(int fmt, RawSource src, int rt, int kc, uint32_t* __restrict__ tiles)
{
    const int words = tile_words(fmt);
    const int64_t total = (int64_t)rt * kc * words;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int w = (int)(i % words);
        const int64_t tile = i / words;
        tiles[i] = repack_tile_word(fmt, src, (int)(tile / kc), (int)(tile % kc), w);
    }
}

__global__ void dequant_packed_kernel(WeightView v, float* __restrict__ out)
{
    const int64_t total = v.n * v.k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        out[i] = dequant_packed_element(v, i / v.k, i % v.k);
    }
}

__global__ void dequant_raw_kernel(int fmt, const uint8_t* __restrict__ payload, int64_t n, int64_t k,
                                   float* __restrict__ out)
{
    const int elems = block_elems(fmt);
    const int bytes = block_bytes(fmt);
    const int64_t total = n * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        // rows are contiguous runs of k/elems blocks, so block index = i / elems
        out[i] = dequant_raw_element(fmt, payload + (i / elems) * bytes, (int)(i % elems));
    }
}

int grid_for(int64_t total, int threads, int sm_count)
{
    int64_t blocks = (total + threads - 1) / threads;
    const int64_t cap = (int64_t)sm_count * 16;
    if (blocks > cap) {
        blocks = cap;
    }
    if (blocks < 1) {
        blocks = 1;
    }
    return (int)blocks;
}

}  // namespace

cudaError_t launch_repack(int fmt, const RawSource& src, int rt, int kc, uint8_t* tiles, int sm_count,
                          cudaStream_t stream)
{
    const int threads = 256;
    const int64_t words = (int64_t)rt * kc * tile_words(fmt);
    repack_kernel<<<grid_for(words, threads, sm_count), threads, 0, stream>>>(fmt, src, rt, kc,
                                                                              reinterpret_cast<uint32_t*>(tiles));
    return cudaGetLastError();
}

cudaError_t launch_dequant_packed(const WeightView& v, float* out, int sm_count, cudaStream_t stream)
{
    const int threads = 256;
    dequant_packed_kernel<<<grid_for(v.n * v.k, threads, sm_count), threads, 0, stream>>>(v, out);
    return cudaGetLastError();
}

cudaError_t launch_dequant_raw(int fmt, const uint8_t* payload, int64_t n, int64_t k, float* out, int sm_count,
                               cudaStream_t stream)
{
    const int threads = 256;
    dequant_raw_kernel<<<grid_for(n * k, threads, sm_count), threads, 0, stream>>>(fmt, payload, n, k, out);
    return cudaGetLastError();
}

}  // namespace qmm

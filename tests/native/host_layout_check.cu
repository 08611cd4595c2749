// Test-only helper: runs the upload-time repack and the packed-layout dequantizer
// on the HOST, through the same __host__ __device__ index functions the CUDA
// kernels call (litenn_b200/csrc/qmm_layout.cuh).  It lets the CPU test suite
// check the tile layout against the oracle without a GPU.  Not part of the
// product library.
#include <cstdint>
#include <vector>

#include "../../litenn_b200/csrc/qmm_layout.cuh"

using namespace qmm;

extern "C" int layout_roundtrip(int fmt, const uint8_t* payload, int64_t full_row_bytes, int64_t row0, int64_t blk0,
                                int64_t n, int64_t k, float* out)
{
    const int elems = block_elems(fmt);
    if (elems == 0 || k % elems != 0) {
        return -1;
    }
    RawSource src;
    src.base = payload;
    src.row_bytes = full_row_bytes;
    src.row0 = row0;
    src.blk0 = blk0;
    src.n = n;
    src.nblk = k / elems;
    const int rt = (int)((n + 15) / 16);
    const int kc = (int)((k + 255) / 256);
    const size_t tiles = (size_t)rt * kc;
    std::vector<uint32_t> packed(tiles * tile_words(fmt));
    for (int r = 0; r < rt; ++r) {
        for (int c = 0; c < kc; ++c) {
            const size_t tile = (size_t)r * kc + c;
            for (int w = 0; w < tile_words(fmt); ++w) {
                packed[tile * tile_words(fmt) + w] = repack_tile_word(fmt, src, r, c, w);
            }
        }
    }
    WeightView v;
    v.tiles = reinterpret_cast<const uint8_t*>(packed.data());
    v.n = n;
    v.k = k;
    v.rt = rt;
    v.kc = kc;
    v.fmt = fmt;
    for (int64_t r = 0; r < n; ++r) {
        for (int64_t c = 0; c < k; ++c) {
            out[r * k + c] = dequant_packed_element(v, r, c);
        }
    }
    return 0;
}

extern "C" int raw_dequant_host(int fmt, const uint8_t* payload, int64_t n, int64_t k, float* out)
{
    const int elems = block_elems(fmt);
    if (elems == 0 || k % elems != 0) {
        return -1;
    }
    for (int64_t i = 0; i < n * k; ++i) {
        out[i] = dequant_raw_element(fmt, payload + (i / elems) * block_bytes(fmt), (int)(i % elems));
    }
    return 0;
}

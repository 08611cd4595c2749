"""Seeded synthetic GGUF block payloads and activations.

Every tensor is drawn from its own counter-based Philox stream keyed by
``(seed, crc32(name))`` so the host oracle, the GPU tests and the bench see
identical bytes regardless of generation order.  Distributions follow the
benchmark configurations: Q8_0 quants uniform in [-127,127] with
d = fp16(|N(0,0.02)|/127); Q4_0 nibbles uniform with d = fp16(|N(0,0.02)|/8);
Q4_K / Q6_K 6-bit scales and quants uniform with d, dmin = fp16(|N(0,0.01)|).

Block byte layouts are the ggml ones that LiteNN's importer keeps as opaque
``UInt8`` payloads (tools/gguf/GGUFImporter.cpp:457-491; block sizes in
src/LiteNN/Quantization.h:186-217).
"""
from __future__ import annotations

import zlib

import numpy as np

# Numeric values of LiteNN::QuantizedBlockFormat (src/LiteNN/Quantization.h:31-62).
Q4_0 = 1
Q8_0 = 5
Q4_K = 9
Q6_K = 11

BLOCK_ELEMS = {Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210}
FORMAT_NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K"}


def rng_for(seed: int, name: str) -> np.random.Generator:
    key = (int(seed) & 0xFFFFFFFF) | ((zlib.crc32(name.encode()) & 0xFFFFFFFF) << 32)
    return np.random.Generator(np.random.Philox(key=key))


def payload_nbytes(fmt: int, n: int, k: int) -> int:
    if k % BLOCK_ELEMS[fmt]:
        raise ValueError(f"K={k} is not a multiple of the {FORMAT_NAMES[fmt]} block size")
    return n * (k // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt]


def _fp16_abs_normal(rng, count, sigma, div):
    vals = np.abs(rng.standard_normal(count, dtype=np.float32) * np.float32(sigma)) / np.float32(div)
    return vals.astype(np.float16).view(np.uint16)


def _put_u16(dst, col, vals):
    dst[:, col] = (vals & 0xFF).astype(np.uint8)
    dst[:, col + 1] = (vals >> 8).astype(np.uint8)


def make_weight(fmt: int, n: int, k: int, seed: int = 0, name: str = "w") -> np.ndarray:
    """Return the raw ggml payload (uint8, ``payload_nbytes`` long) of a ``[n, k]`` weight."""
    rng = rng_for(seed, name)
    nblk = n * (k // BLOCK_ELEMS[fmt])
    out = np.empty((nblk, BLOCK_BYTES[fmt]), dtype=np.uint8)
    if fmt == Q8_0:
        _put_u16(out, 0, _fp16_abs_normal(rng, nblk, 0.02, 127.0))
        out[:, 2:] = rng.integers(-127, 128, size=(nblk, 32), dtype=np.int8).view(np.uint8)
    elif fmt == Q4_0:
        _put_u16(out, 0, _fp16_abs_normal(rng, nblk, 0.02, 8.0))
        out[:, 2:] = rng.integers(0, 256, size=(nblk, 16), dtype=np.uint8)
    elif fmt == Q4_K:
        _put_u16(out, 0, _fp16_abs_normal(rng, nblk, 0.01, 1.0))
        _put_u16(out, 2, _fp16_abs_normal(rng, nblk, 0.01, 1.0))
        # 12 bytes of packed 6-bit (scale, min) pairs: every bit pattern is a
        # valid encoding and uniform bytes give uniform 6-bit fields.
        out[:, 4:16] = rng.integers(0, 256, size=(nblk, 12), dtype=np.uint8)
        out[:, 16:] = rng.integers(0, 256, size=(nblk, 128), dtype=np.uint8)
    elif fmt == Q6_K:
        out[:, 0:192] = rng.integers(0, 256, size=(nblk, 192), dtype=np.uint8)
        out[:, 192:208] = rng.integers(-128, 128, size=(nblk, 16), dtype=np.int8).view(np.uint8)
        _put_u16(out, 208, _fp16_abs_normal(rng, nblk, 0.01, 1.0))
    else:
        raise ValueError(f"unsupported block format {fmt}")
    return out.reshape(-1)


def make_activation(m: int, k: int, seed: int = 0, name: str = "x") -> np.ndarray:
    """fp32 ``[m, k]`` activations ~ N(0,1)."""
    return rng_for(seed, name).standard_normal((m, k), dtype=np.float32)


def make_token_ids(count: int, vocab: int, seed: int = 0, name: str = "prompt") -> np.ndarray:
    return rng_for(seed, name).integers(0, vocab, size=count, dtype=np.int32)


def make_norm_weight(d: int, seed: int = 0, name: str = "norm") -> np.ndarray:
    """RMSNorm weights ~ N(1, 0.1), fp32 ``[d]`` (trained norms sit near one without being one)."""
    return (1.0 + 0.1 * rng_for(seed, name).standard_normal(d, dtype=np.float32)).astype(np.float32)

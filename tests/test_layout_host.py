"""The upload-time repack layout, exercised on the host.

The index functions the repack and dequant kernels call are __host__ __device__;
tests/native/host_layout_check.cu drives them on the CPU so the tile layout is
proved against the oracle (bit-exact, whole tensors and tensor-parallel shards)
without a GPU.  Needs nvcc to compile the helper.
"""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

import oracle
from litenn_b200 import synth
from helpers import FORMATS, assert_bit_exact, random_payload

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "native", "host_layout_check.cu")
OUT = os.path.join(HERE, "native", "liblayout_check.so")


@pytest.fixture(scope="module")
def checker():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    deps = [SRC] + [os.path.join(HERE, "..", "litenn_b200", "csrc", f) for f in ("qmm_layout.cuh", "qmm_common.cuh")]
    if not os.path.exists(OUT) or any(os.path.getmtime(d) > os.path.getmtime(OUT) for d in deps):
        cmd = [nvcc, "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-shared", "-Xcompiler", "-fPIC", "-o", OUT,
               SRC]
        if os.path.exists("/usr/bin/g++"):
            cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
        subprocess.run(cmd, check=True)
    L = ctypes.CDLL(OUT)
    L.layout_roundtrip.argtypes = [ctypes.c_int, ctypes.c_void_p] + [ctypes.c_int64] * 5 + [ctypes.c_void_p]
    L.raw_dequant_host.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
    return L


def roundtrip(L, fmt, payload, full_k, row0, blk0, n, k):
    out = np.empty((n, k), dtype=np.float32)
    row_bytes = (full_k // synth.BLOCK_ELEMS[fmt]) * synth.BLOCK_BYTES[fmt]
    assert L.layout_roundtrip(fmt, payload.ctypes.data, row_bytes, row0, blk0, n, k, out.ctypes.data) == 0
    return out


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(16, 256), (24, 512), (40, 768), (7, 1024), (33, 2048)])
def test_repack_then_dequant_matches_oracle(checker, fmt, shape):
    n, k = shape
    payload = random_payload(fmt, n, k, seed=n * 1000 + k + fmt)
    ref = oracle.dequant(fmt, payload, n, k)
    assert_bit_exact(roundtrip(checker, fmt, payload, k, 0, 0, n, k), ref, "packed")
    raw = np.empty((n, k), dtype=np.float32)
    assert checker.raw_dequant_host(fmt, payload.ctypes.data, n, k, raw.ctypes.data) == 0
    assert_bit_exact(raw, ref, "raw")


@pytest.mark.parametrize("fmt", [synth.Q4_0, synth.Q8_0])
def test_ragged_k_small_blocks(checker, fmt):
    """K that is a multiple of 32 but not of the 256-wide tile (e.g. 11008/8 = 1376)."""
    for n, k in [(5, 96), (18, 1376), (16, 32)]:
        payload = random_payload(fmt, n, k, seed=k + fmt)
        assert_bit_exact(roundtrip(checker, fmt, payload, k, 0, 0, n, k), oracle.dequant(fmt, payload, n, k), "ragged")


@pytest.mark.parametrize("fmt", FORMATS)
def test_shards(checker, fmt):
    n, k, tp = 48, 2048, 4
    payload = random_payload(fmt, n, k, seed=99 + fmt)
    ref = oracle.dequant(fmt, payload, n, k)
    for rank in range(tp):
        rows = n // tp
        got = roundtrip(checker, fmt, payload, k, rank * rows, 0, rows, k)
        assert_bit_exact(got, ref[rank * rows:(rank + 1) * rows], f"N shard {rank}")
        cols = k // tp
        blk0 = (cols // synth.BLOCK_ELEMS[fmt]) * rank
        got = roundtrip(checker, fmt, payload, k, 0, blk0, n, cols)
        assert_bit_exact(got, ref[:, rank * cols:(rank + 1) * cols], f"K shard {rank}")


@pytest.mark.parametrize("name,fmt", [("q4_1", 2), ("q5_0", 3), ("q5_1", 4), ("q2_k", 7), ("q3_k", 8), ("q5_k", 10)])
def test_carried_formats_raw_dequant_on_the_host(checker, name, fmt):
    """The device code's element function for the formats that are only dequantized, run on the CPU: bit-exact
    with the committed ggml-py goldens."""
    g = np.load(os.path.join(HERE, "golden", "dequant_carried_golden.npz"))
    n, k = int(g["rows"]), int(g["k"])
    payload = np.ascontiguousarray(g[name + "_payload"])
    raw = np.empty((n, k), dtype=np.float32)
    assert checker.raw_dequant_host(fmt, payload.ctypes.data, n, k, raw.ctypes.data) == 0
    assert_bit_exact(raw, g[name + "_values"], name)

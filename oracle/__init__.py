"""ctypes access to the CPU oracle (``libqmm_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  Nothing
in the product package may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqmm_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only)."""
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".c", ".h"))]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-s", "-B"], check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.oracle_block_elems.argtypes = [ci]
        L.oracle_block_bytes.argtypes = [ci]
        L.oracle_fp16_to_fp32.argtypes = [ctypes.c_uint16]
        L.oracle_fp16_to_fp32.restype = ctypes.c_float
        L.oracle_fp32_to_fp16.argtypes = [ctypes.c_float]
        L.oracle_fp32_to_fp16.restype = ctypes.c_uint16
        L.oracle_fp32_to_bf16.argtypes = [ctypes.c_float]
        L.oracle_fp32_to_bf16.restype = ctypes.c_uint16
        L.oracle_bf16_to_fp32.argtypes = [ctypes.c_uint16]
        L.oracle_bf16_to_fp32.restype = ctypes.c_float
        L.oracle_dequant.argtypes = [ci, vp, i64, i64, vp]
        L.oracle_dequant.restype = ci
        L.oracle_transpose.argtypes = [vp, i64, i64, vp]
        L.oracle_transpose.restype = None
        L.oracle_matmul_ikj.argtypes = [vp, vp, vp, i64, i64, i64]
        L.oracle_matmul_ikj.restype = None
        L.oracle_matmul_ikj_mt.argtypes = [vp, vp, vp, i64, i64, i64, ci]
        L.oracle_matmul_ikj_mt.restype = None
        L.oracle_matmul_nk.argtypes = [vp, vp, vp, i64, i64, i64, ci]
        L.oracle_matmul_nk.restype = None
        L.oracle_matmul_nk_f64.argtypes = [vp, vp, vp, i64, i64, i64, ci]
        L.oracle_matmul_nk_f64.restype = None
        L.oracle_max_threads.restype = ci
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def dequant(fmt: int, payload: np.ndarray, n: int, k: int) -> np.ndarray:
    """fp32 ``[n, k]`` values of a raw ggml payload (LLaMABuilder.cpp:66-162)."""
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    elems, nbytes = lib().oracle_block_elems(fmt), lib().oracle_block_bytes(fmt)
    if elems == 0:
        raise ValueError(f"unknown block format {fmt}")
    if k % elems:
        raise ValueError(f"row width {k} is incompatible with block size {elems}")
    if payload.size != n * (k // elems) * nbytes:
        raise ValueError("payload byte count does not match the expressed shape")
    out = np.empty((n, k), dtype=np.float32)
    rc = lib().oracle_dequant(fmt, _ptr(payload), n, k, _ptr(out))
    if rc != 0:
        raise ValueError(f"oracle_dequant failed with {rc}")
    return out


def transpose(w: np.ndarray) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty((w.shape[1], w.shape[0]), dtype=np.float32)
    lib().oracle_transpose(_ptr(w), w.shape[0], w.shape[1], _ptr(out))
    return out


def matmul_ikj(x: np.ndarray, wt: np.ndarray, threads: int = 1) -> np.ndarray:
    """The reference MatMul loop (Device.h:645-658) on ``x[M,K] @ wt[K,N]``."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    wt = np.ascontiguousarray(wt, dtype=np.float32)
    m, k = x.shape
    assert wt.shape[0] == k
    n = wt.shape[1]
    out = np.empty((m, n), dtype=np.float32)
    if threads <= 1:
        lib().oracle_matmul_ikj(_ptr(x), _ptr(wt), _ptr(out), m, k, n)
    else:
        lib().oracle_matmul_ikj_mt(_ptr(x), _ptr(wt), _ptr(out), m, k, n, threads)
    return out


def matmul_nk(x: np.ndarray, w: np.ndarray, threads: int = 0) -> np.ndarray:
    """Bit-identical to :func:`matmul_ikj` on the transposed weight, reading ``w[N,K]``."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k
    out = np.empty((m, n), dtype=np.float32)
    lib().oracle_matmul_nk(_ptr(x), _ptr(w), _ptr(out), m, k, n, threads or max_threads())
    return out


def matmul_nk_f64(x: np.ndarray, w: np.ndarray, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    m, k = x.shape
    n = w.shape[0]
    out = np.empty((m, n), dtype=np.float64)
    lib().oracle_matmul_nk_f64(_ptr(x), _ptr(w), _ptr(out), m, k, n, threads or max_threads())
    return out


def quantized_matmul(fmt: int, payload: np.ndarray, n: int, k: int, x: np.ndarray, threads: int = 0) -> np.ndarray:
    """Reference result of the quantized linear: dequantize, then the fp32 loop."""
    return matmul_nk(x, dequant(fmt, payload, n, k), threads)


def fp32_to_bf16_round(a: np.ndarray) -> np.ndarray:
    """Round fp32 values to bf16 (nearest even) and return them as fp32."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = ((bits + 0x7FFF + lsb) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(a.shape)

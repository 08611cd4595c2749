"""ctypes binding of the C ABI in ``include/litenn_qmm.h``.

This is the Python-side stub a maintainer would use from test or tooling code;
the C++ adapter under ``litenn_b200/host`` is the LiteNN-facing one.  Device
memory is addressed by raw pointers (``torch.Tensor.data_ptr()`` in the tests).
The library has no CPU fallback: when ``libqmm_b200.so`` is missing, loading
fails with an error instead of routing anywhere else.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqmm_b200.so")

Q4_0, Q8_0, Q4_K, Q6_K = 1, 5, 9, 11
SPLIT_NONE, SPLIT_N, SPLIT_K = 0, 1, 2
OUT_F32, OUT_BF16 = 0, 1
GEMV_MAX_BATCH = 16

E_INVALID, E_CUDA, E_UNSUPPORTED, E_KERNEL = -1, -2, -3, -4


class QmmError(RuntimeError):
    """Raised for a non-zero status; mirrors LiteNN's std::runtime_error convention."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class WeightInfo(ctypes.Structure):
    _fields_ = [
        ("fmt", ctypes.c_int32),
        ("device", ctypes.c_int32),
        ("n", ctypes.c_int64),
        ("k", ctypes.c_int64),
        ("payload_bytes", ctypes.c_int64),
        ("packed_bytes", ctypes.c_int64),
    ]


# name -> (restype, argtypes); every symbol include/litenn_qmm.h declares.
_vp, _i, _i64, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
SYMBOLS = {
    "qmm_abi_version": (_i, []),
    "qmm_last_error": (ctypes.c_char_p, []),
    "qmm_block_layout": (_i, [_i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "qmm_device_count": (_i, []),
    "qmm_weight_create": (_i, [_i, _i, _vp, _sz, _i, _i64, _i64, _vp, ctypes.POINTER(_vp)]),
    "qmm_weight_create_shard": (_i, [_i, _i, _vp, _sz, _i, _i64, _i64, _i, _i, _i, _vp, ctypes.POINTER(_vp)]),
    "qmm_weight_destroy": (_i, [_vp]),
    "qmm_weight_get_info": (_i, [_vp, ctypes.POINTER(WeightInfo)]),
    "qmm_dequantize": (_i, [_vp, _vp, _vp]),
    "qmm_dequantize_raw": (_i, [_i, _i, _vp, _i64, _i64, _vp, _vp]),
    "qmm_gemv_f32": (_i, [_vp, _vp, _vp, _i, _vp]),
    "qmm_gemv_f32_static": (_i, [_vp, _vp, _vp, _i, _vp]),
    "qmm_packed_activation_bytes": (_i, [_i64, _i, ctypes.POINTER(_sz)]),
    "qmm_pack_activations": (_i, [_i, _vp, _i, _i64, _vp, _vp]),
    "qmm_gemv_packed": (_i, [_vp, _vp, _vp, _i, _vp]),
    "qmm_unpack_activations": (_i, [_i, _vp, _i64, _vp, _vp]),
    "qmm_gemv_packed_rms": (_i, [_vp, _vp, _vp, _i, _i64, ctypes.c_float, _vp, _vp]),
    "qmm_gemv_packed_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "qmm_gemv_f32_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "qmm_gemv_packed_swiglu": (_i, [_vp, _vp, _vp, _i, _i64, ctypes.c_float, _vp, _vp]),
    "qmm_gemv_packed_swiglu_pack": (_i, [_vp, _vp, _vp, _i, _i64, ctypes.c_float, _vp, _vp, _vp]),
    "qmm_interleave_gate_up": (_i, [_i, _vp, _vp, _i64, _i64, _vp]),
    "qmm_gemm_bf16": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "qmm_gemm_f32": (_i, [_vp, _vp, _vp, _i64, _vp]),
    "qmm_gemv_f32_host": (_i, [_vp, _vp, _vp, _i, _vp]),
    "qmm_kernel_status": (_i, [_i, ctypes.POINTER(_i)]),
    "qmm_stream_synchronize": (_i, [_i, _vp]),
    "qmm_release_workspaces": (_i, []),
}



class LlamaConfig(ctypes.Structure):
    """Mirror of qmm_llama_config (include/litenn_llama.h)."""
    _fields_ = [(n, ctypes.c_int32) for n in (
        "n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "rope_dim", "max_seq",
        "max_prefill", "tp_rank", "tp_size", "embd_fmt")] + [("rms_eps", ctypes.c_float), ("rope_theta", ctypes.c_float)]


# include/litenn_llama.h
LLAMA_SYMBOLS = {
    "qmm_llama_create": (_i, [_i, ctypes.POINTER(LlamaConfig), ctypes.POINTER(_vp)]),
    "qmm_llama_destroy": (_i, [_vp]),
    "qmm_llama_set_weight": (_i, [_vp, _i, _i, _vp]),
    "qmm_llama_set_norm": (_i, [_vp, _i, _i, _vp]),
    "qmm_llama_set_embedding": (_i, [_vp, _vp, _sz]),
    "qmm_llama_tp_unique_id": (_i, [ctypes.c_char_p, ctypes.c_char_p]),
    "qmm_llama_tp_init": (_i, [_vp, ctypes.c_char_p, ctypes.c_char_p]),
    "qmm_llama_tp_export": (_i, [_vp, ctypes.c_char_p]),
    "qmm_llama_tp_import": (_i, [_vp, ctypes.c_char_p, _vp]),
    "qmm_llama_reset": (_i, [_vp, _vp]),
    "qmm_llama_prefill": (_i, [_vp, _vp, _i, ctypes.POINTER(ctypes.c_int32), _vp]),
    "qmm_llama_decode": (_i, [_vp, _i, _vp, _vp]),
    "qmm_llama_decode_enqueue": (_i, [_vp, _i, _vp]),
    "qmm_llama_step_host": (_i, [_vp, ctypes.c_int32, ctypes.POINTER(ctypes.c_int32), _vp]),
    "qmm_llama_last_logits": (_i, [_vp, _vp, _vp]),
    "qmm_llama_tie_output": (_i, [_vp, _vp, _sz, _vp]),
    "qmm_llama_set_wait_limit": (_i, [_vp, ctypes.c_uint]),
    "qmm_llama_set_collective_timeout": (_i, [_vp, _i]),
    "qmm_llama_tp_loopback": (_i, [_vp]),
    "qmm_llama_has_graph": (_i, [_vp]),
    "qmm_llama_generated_tokens": (_i, [_vp, _i, _i, _vp, _vp]),
    "qmm_llama_batch_create": (_i, [_vp, _i, _i]),
    "qmm_llama_batch_prefill": (_i, [_vp, _i, _vp, _i, _vp, _vp]),
    "qmm_llama_batch_decode": (_i, [_vp, _i, _vp, _vp]),
    "qmm_llama_batch_decode_enqueue": (_i, [_vp, _i, _vp]),
    "qmm_llama_batch_generated_tokens": (_i, [_vp, _i, _i, _vp, _vp]),
}
LL_QKV, LL_O, LL_GU, LL_DOWN, LL_HEAD = 0, 1, 2, 3, 4
LL_ATTN_NORM, LL_FFN_NORM, LL_FINAL_NORM = 0, 1, 2

_lib = None


def load() -> ctypes.CDLL:
    """Load the library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m litenn_b200.build` "
                "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for this path.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in {**SYMBOLS, **LLAMA_SYMBOLS}.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    return load().qmm_last_error().decode(errors="replace")


def check(rc: int) -> None:
    if rc != 0:
        raise QmmError(rc, last_error())


def block_layout(fmt: int) -> tuple[int, int]:
    e, b = ctypes.c_int(), ctypes.c_int()
    check(load().qmm_block_layout(fmt, ctypes.byref(e), ctypes.byref(b)))
    return e.value, b.value


def device_count() -> int:
    return int(load().qmm_device_count())


class Weight:
    """Owns one ``qmm_weight`` handle (a packed, device-resident quantized tensor)."""

    def __init__(self, handle: int):
        self._h = ctypes.c_void_p(handle)

    @classmethod
    def from_host(cls, fmt: int, payload, n: int, k: int, device: int = 0, stream: int = 0,
                  split: int = SPLIT_NONE, tp_rank: int = 0, tp_size: int = 1) -> "Weight":
        """`payload` is a contiguous uint8 numpy array holding the raw ggml blocks."""
        h = ctypes.c_void_p()
        ptr = ctypes.c_void_p(payload.ctypes.data)
        if split == SPLIT_NONE:
            rc = load().qmm_weight_create(device, fmt, ptr, payload.nbytes, 0, n, k, ctypes.c_void_p(stream),
                                          ctypes.byref(h))
        else:
            rc = load().qmm_weight_create_shard(device, fmt, ptr, payload.nbytes, 0, n, k, split, tp_rank, tp_size,
                                                ctypes.c_void_p(stream), ctypes.byref(h))
        check(rc)
        return cls(h.value)

    @classmethod
    def from_device(cls, fmt: int, payload_ptr: int, payload_bytes: int, n: int, k: int, device: int = 0,
                    stream: int = 0, split: int = SPLIT_NONE, tp_rank: int = 0, tp_size: int = 1) -> "Weight":
        h = ctypes.c_void_p()
        rc = load().qmm_weight_create_shard(device, fmt, ctypes.c_void_p(payload_ptr), payload_bytes, 1, n, k, split,
                                            tp_rank, tp_size, ctypes.c_void_p(stream), ctypes.byref(h))
        check(rc)
        return cls(h.value)

    @property
    def handle(self) -> ctypes.c_void_p:
        if not self._h:
            raise QmmError(E_INVALID, "weight handle already destroyed")
        return self._h

    def info(self) -> WeightInfo:
        out = WeightInfo()
        check(load().qmm_weight_get_info(self.handle, ctypes.byref(out)))
        return out

    def dequantize(self, out_ptr: int, stream: int = 0) -> None:
        check(load().qmm_dequantize(self.handle, ctypes.c_void_p(out_ptr), ctypes.c_void_p(stream)))

    def gemv_f32(self, x_ptr: int, y_ptr: int, m: int, stream: int = 0) -> None:
        check(load().qmm_gemv_f32(self.handle, ctypes.c_void_p(x_ptr), ctypes.c_void_p(y_ptr), m,
                                  ctypes.c_void_p(stream)))

    def gemv_f32_static(self, x_ptr: int, y_ptr: int, m: int, stream: int = 0) -> None:
        """qmm_gemv_f32 without any device allocation (fixed scratch inside the library)."""
        check(load().qmm_gemv_f32_static(self.handle, ctypes.c_void_p(x_ptr), ctypes.c_void_p(y_ptr), m,
                                         ctypes.c_void_p(stream)))

    def gemv_packed(self, packed_ptr: int, y_ptr: int, m: int, stream: int = 0) -> None:
        check(load().qmm_gemv_packed(self.handle, ctypes.c_void_p(packed_ptr), ctypes.c_void_p(y_ptr), m,
                                     ctypes.c_void_p(stream)))

    def gemv_packed_rms(self, packed_ptr: int, ss_ptr: int, ss_count: int, d_in: int, eps: float, y_ptr: int,
                        stream: int = 0) -> None:
        check(load().qmm_gemv_packed_rms(self.handle, ctypes.c_void_p(packed_ptr), ctypes.c_void_p(ss_ptr), ss_count,
                                         d_in, eps, ctypes.c_void_p(y_ptr), ctypes.c_void_p(stream)))

    def gemv_packed_residual(self, packed_ptr: int, h_ptr: int, norm_w_ptr: int, packed_out_ptr: int, ss_out_ptr: int,
                             stream: int = 0) -> None:
        check(load().qmm_gemv_packed_residual(self.handle, ctypes.c_void_p(packed_ptr), ctypes.c_void_p(h_ptr),
                                              ctypes.c_void_p(norm_w_ptr), ctypes.c_void_p(packed_out_ptr),
                                              ctypes.c_void_p(ss_out_ptr), ctypes.c_void_p(stream)))

    def gemv_f32_residual(self, x_ptr: int, h_ptr: int, norm_w_ptr: int, packed_out_ptr: int, ss_out_ptr: int,
                          stream: int = 0) -> None:
        check(load().qmm_gemv_f32_residual(self.handle, ctypes.c_void_p(x_ptr), ctypes.c_void_p(h_ptr),
                                           ctypes.c_void_p(norm_w_ptr), ctypes.c_void_p(packed_out_ptr),
                                           ctypes.c_void_p(ss_out_ptr), ctypes.c_void_p(stream)))

    def gemv_packed_swiglu(self, packed_ptr: int, ss_ptr: int, ss_count: int, d_in: int, eps: float, act_ptr: int,
                           stream: int = 0) -> None:
        check(load().qmm_gemv_packed_swiglu(self.handle, ctypes.c_void_p(packed_ptr), ctypes.c_void_p(ss_ptr or None),
                                            ss_count, d_in, eps, ctypes.c_void_p(act_ptr), ctypes.c_void_p(stream)))

    def gemv_packed_swiglu_pack(self, packed_ptr: int, ss_ptr: int, ss_count: int, d_in: int, eps: float,
                                packed_out_ptr: int, act_ptr: int = 0, stream: int = 0) -> None:
        check(load().qmm_gemv_packed_swiglu_pack(self.handle, ctypes.c_void_p(packed_ptr), ctypes.c_void_p(ss_ptr or None),
                                                 ss_count, d_in, eps, ctypes.c_void_p(packed_out_ptr),
                                                 ctypes.c_void_p(act_ptr or None), ctypes.c_void_p(stream)))

    def gemv_f32_host(self, x_host, y_host, m: int, stream: int = 0) -> None:
        """`x_host`, `y_host`: contiguous fp32 numpy arrays (ideally pinned)."""
        check(load().qmm_gemv_f32_host(self.handle, ctypes.c_void_p(x_host.ctypes.data),
                                       ctypes.c_void_p(y_host.ctypes.data), m, ctypes.c_void_p(stream)))

    def gemm_bf16(self, x_ptr: int, y_ptr: int, m: int, out_dtype: int = OUT_F32, stream: int = 0) -> None:
        check(load().qmm_gemm_bf16(self.handle, ctypes.c_void_p(x_ptr), ctypes.c_void_p(y_ptr), m, out_dtype,
                                   ctypes.c_void_p(stream)))

    def gemm_f32(self, x_ptr: int, y_ptr: int, m: int, stream: int = 0) -> None:
        """fp32 activations of any row count through the prefill GEMM (rounded to bf16 on the device)."""
        check(load().qmm_gemm_f32(self.handle, ctypes.c_void_p(x_ptr), ctypes.c_void_p(y_ptr), m,
                                  ctypes.c_void_p(stream)))

    def destroy(self) -> None:
        if self._h:
            h, self._h = self._h, ctypes.c_void_p()
            check(load().qmm_weight_destroy(h))

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def dequantize_raw(fmt: int, payload_ptr: int, n: int, k: int, out_ptr: int, device: int = 0, stream: int = 0) -> None:
    check(load().qmm_dequantize_raw(device, fmt, ctypes.c_void_p(payload_ptr), n, k, ctypes.c_void_p(out_ptr),
                                    ctypes.c_void_p(stream)))


def packed_activation_bytes(k: int, m: int) -> int:
    out = ctypes.c_size_t()
    check(load().qmm_packed_activation_bytes(k, m, ctypes.byref(out)))
    return out.value


def pack_activations(x_ptr: int, m: int, k: int, packed_ptr: int, device: int = 0, stream: int = 0) -> None:
    check(load().qmm_pack_activations(device, ctypes.c_void_p(x_ptr), m, k, ctypes.c_void_p(packed_ptr),
                                      ctypes.c_void_p(stream)))


def unpack_activations(packed_ptr: int, k: int, x_ptr: int, device: int = 0, stream: int = 0) -> None:
    check(load().qmm_unpack_activations(device, ctypes.c_void_p(packed_ptr), k, ctypes.c_void_p(x_ptr),
                                        ctypes.c_void_p(stream)))


def interleave_gate_up(fmt: int, gate, up, n_each: int, k: int):
    """Raw payloads of ffn_gate and ffn_up -> one payload alternating 8 rows of gate, 8 rows of up."""
    import numpy as np
    out = np.empty(gate.nbytes + up.nbytes, dtype=np.uint8)
    check(load().qmm_interleave_gate_up(fmt, ctypes.c_void_p(gate.ctypes.data), ctypes.c_void_p(up.ctypes.data),
                                        n_each, k, ctypes.c_void_p(out.ctypes.data)))
    return out


def kernel_status(device: int = 0) -> int:
    """Synchronizes with `device`; raises QmmError(E_KERNEL) if a kernel gave up on a bounded wait."""
    st = ctypes.c_int(0)
    check(load().qmm_kernel_status(device, ctypes.byref(st)))
    return st.value


def release_workspaces() -> None:
    check(load().qmm_release_workspaces())

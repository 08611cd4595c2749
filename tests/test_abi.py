"""The C-ABI library loads without a GPU and exports what include/litenn_qmm.h declares."""
import ctypes
import os
import re

import numpy as np
import pytest

from litenn_b200 import capi, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="litenn_qmm.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qmm_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_symbols()
    assert names, "no declarations found"
    assert sorted(capi.SYMBOLS) == names


def test_library_exports_every_declared_symbol(qmm_lib):
    for name in declared_symbols():
        assert hasattr(qmm_lib, name), name
    assert qmm_lib.qmm_abi_version() == 2


def test_decoder_header_and_binding_agree(qmm_lib):
    names = declared_symbols("litenn_llama.h")
    assert names, "no declarations found"
    assert sorted(capi.LLAMA_SYMBOLS) == names
    for name in names:
        assert hasattr(qmm_lib, name), name


def test_decoder_rejects_bad_arguments_without_a_gpu(qmm_lib):
    assert qmm_lib.qmm_llama_set_wait_limit(None, 1) == capi.E_INVALID
    assert qmm_lib.qmm_llama_has_graph(None) == 0
    assert qmm_lib.qmm_llama_destroy(None) == 0
    cfg = capi.LlamaConfig(1, 256, 4, 2, 96, 512, 512, 96, 64, 32, 0, 1, capi.Q6_K, 1e-6, 10000.0)
    h = ctypes.c_void_p()
    assert qmm_lib.qmm_llama_create(0, ctypes.byref(cfg), ctypes.byref(h)) == capi.E_INVALID  # head_dim 96


def test_block_layout(qmm_lib):
    # src/LiteNN/Quantization.h:186-217
    assert capi.block_layout(capi.Q4_0) == (32, 18)
    assert capi.block_layout(capi.Q8_0) == (32, 34)
    assert capi.block_layout(capi.Q4_K) == (256, 144)
    assert capi.block_layout(capi.Q6_K) == (256, 210)
    # carried formats (dequantized, never multiplied): Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K by LiteNN's enum values
    assert [capi.block_layout(f) for f in (2, 3, 4, 7, 8, 10)] == [(32, 20), (32, 22), (32, 24), (256, 84), (256, 110),
                                                                  (256, 176)]
    with pytest.raises(capi.QmmError) as e:
        capi.block_layout(6)      # Q8_1: an activation format, not a tensor format of the importer
    assert e.value.code == capi.E_UNSUPPORTED
    with pytest.raises(capi.QmmError) as e:   # a carried format has a layout but no packed weight
        capi.Weight.from_host(2, np.zeros(20, dtype=np.uint8), 1, 32)
    assert e.value.code == capi.E_UNSUPPORTED


def test_argument_validation_needs_no_gpu(qmm_lib):
    """Shape errors are reported before any CUDA call, with LiteNN-style messages
    (tools/gguf/LLaMABuilder.cpp:121-126, 137-142)."""
    payload = np.zeros(18 * 3, dtype=np.uint8)
    with pytest.raises(capi.QmmError) as e:
        capi.Weight.from_host(capi.Q4_0, payload, 1, 80)
    assert e.value.code == capi.E_INVALID and "incompatible with ggml block size" in str(e.value)
    with pytest.raises(capi.QmmError) as e:
        capi.Weight.from_host(capi.Q4_0, payload, 2, 64)
    assert e.value.code == capi.E_INVALID and "does not match expressed shape" in str(e.value)
    with pytest.raises(capi.QmmError) as e:
        capi.Weight.from_host(3, payload, 1, 96)
    assert e.value.code == capi.E_UNSUPPORTED
    # K shards must be whole blocks and must never be truncated: 11008/256 = 43 super-blocks
    big = np.zeros(synth.payload_nbytes(capi.Q4_K, 1, 11008), dtype=np.uint8)
    with pytest.raises(capi.QmmError) as e:
        capi.Weight.from_host(capi.Q4_K, big, 1, 11008, split=capi.SPLIT_K, tp_rank=0, tp_size=2)
    assert e.value.code == capi.E_INVALID and "whole" in str(e.value)
    with pytest.raises(capi.QmmError) as e:
        capi.Weight.from_host(capi.Q4_0, payload, 3, 32, split=capi.SPLIT_N, tp_rank=0, tp_size=2)
    assert e.value.code == capi.E_INVALID


def test_no_cpu_fallback(qmm_lib):
    """Without a CUDA device the compute path fails loudly instead of falling back."""
    if capi.device_count() > 0:
        pytest.skip("a GPU is present")
    payload = synth.make_weight(capi.Q4_0, 16, 256)
    with pytest.raises(capi.QmmError) as e:
        capi.Weight.from_host(capi.Q4_0, payload, 16, 256)
    assert e.value.code == capi.E_CUDA


def test_gate_up_interleave_is_a_row_permutation(qmm_lib):
    """qmm_interleave_gate_up is host-only: 8 rows of gate, the same 8 rows of up, and so on."""
    n, k = 24, 64
    gate = synth.make_weight(capi.Q4_0, n, k, seed=1, name="il.gate")
    up = synth.make_weight(capi.Q4_0, n, k, seed=1, name="il.up")
    out = capi.interleave_gate_up(capi.Q4_0, gate, up, n, k)
    rb = k // 32 * 18
    g, u, o = gate.reshape(n, rb), up.reshape(n, rb), out.reshape(2 * n, rb)
    for c in range(n):
        assert np.array_equal(o[(c // 8) * 16 + c % 8], g[c])
        assert np.array_equal(o[(c // 8) * 16 + 8 + c % 8], u[c])
    with pytest.raises(capi.QmmError):
        capi.interleave_gate_up(capi.Q4_0, gate, up, 20, k)  # not a multiple of 8


def test_null_handles_are_rejected(qmm_lib):
    assert qmm_lib.qmm_gemv_f32(None, None, None, 1, None) == capi.E_INVALID
    assert "null" in capi.last_error()
    assert qmm_lib.qmm_weight_destroy(None) == 0


def test_product_package_never_touches_the_oracle():
    """The oracle is test infrastructure; the package must not import or load it."""
    pkg = os.path.join(ROOT, "litenn_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
                assert "qmm_oracle" not in text, f

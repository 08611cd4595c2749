"""The CPU oracle against the reference's own fixtures and the golden vectors."""
import numpy as np
import pytest

import oracle
from litenn_b200 import synth
from helpers import FORMATS, assert_bit_exact


def test_block_layout_table():
    # src/LiteNN/Quantization.h:186-217
    L = oracle.lib()
    assert (L.oracle_block_elems(synth.Q4_0), L.oracle_block_bytes(synth.Q4_0)) == (32, 18)
    assert (L.oracle_block_elems(synth.Q8_0), L.oracle_block_bytes(synth.Q8_0)) == (32, 34)
    assert (L.oracle_block_elems(synth.Q4_K), L.oracle_block_bytes(synth.Q4_K)) == (256, 144)
    assert (L.oracle_block_elems(synth.Q6_K), L.oracle_block_bytes(synth.Q6_K)) == (256, 210)
    # carried formats (dequantized only): Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K
    assert [(L.oracle_block_elems(f), L.oracle_block_bytes(f)) for f in (2, 3, 4, 7, 8, 10)] == [
        (32, 20), (32, 22), (32, 24), (256, 84), (256, 110), (256, 176)]
    assert L.oracle_block_elems(6) == 0  # Q8_1: an activation format, not a tensor format of the importer


def test_reference_q4_0_fixture():
    """The 18-byte Q4_0 payload of tests/GGUFImporterTest.cpp:173-176 (d = fp16 0x0010 = 2^-20)."""
    payload = np.array([0x10, 0x00, 0x22, 0x44, 0x66, 0x88, 0xaa, 0xcc, 0xee, 0x11, 0x33, 0x55, 0x77, 0x99,
                        0xbb, 0xdd, 0xff, 0x7f], dtype=np.uint8)
    assert payload[0] == 0x10 and payload[17] == 0x7f and payload.size == 18
    got = oracle.dequant(synth.Q4_0, payload, 1, 32)[0]
    d = np.float32(2.0 ** -20)
    low = np.array([-6, -4, -2, 0, 2, 4, 6, -7, -5, -3, -1, 1, 3, 5, 7, 7], dtype=np.float32)
    high = np.array([-6, -4, -2, 0, 2, 4, 6, -7, -5, -3, -1, 1, 3, 5, 7, -1], dtype=np.float32)
    assert_bit_exact(got, np.concatenate([low, high]) * d, "Q4_0 reference fixture")


@pytest.mark.parametrize("fmt", FORMATS)
def test_golden_vectors(golden, fmt):
    """Bit-exact with the ggml project's Python dequantizers on committed random payloads."""
    name = synth.FORMAT_NAMES[fmt]
    n, k = int(golden["rows"]), int(golden["k"])
    for variant in ("", "_syn"):
        got = oracle.dequant(fmt, golden[f"{name}{variant}_payload"], n, k)
        assert_bit_exact(got, golden[f"{name}{variant}_values"], f"{name}{variant}")


def test_synthetic_generator_is_stable(golden):
    """The seeded generator reproduces the bytes the fixtures were made from."""
    n, k = int(golden["rows"]), int(golden["k"])
    for fmt in FORMATS:
        name = synth.FORMAT_NAMES[fmt]
        again = synth.make_weight(fmt, n, k, seed=7, name="golden-syn-" + name)
        assert np.array_equal(again, golden[f"{name}_syn_payload"])


def test_zero_weights_dequantize_to_zero():
    """What GGUFLLaMACausalLM.LowersQuantizedWeightsByDequantizingDuringImport pins
    (tests/GGUFImporterTest.cpp:1037-1067): quantized zeros come back as zeros."""
    blk = np.zeros(34, dtype=np.uint8)  # Q8_0: d = 0, q = 0
    assert not oracle.dequant(synth.Q8_0, np.tile(blk, 4), 2, 64).any()


def test_fp16_conversions_match_numpy():
    L = oracle.lib()
    all_bits = np.arange(65536, dtype=np.uint16)
    ref = all_bits.view(np.float16).astype(np.float32)
    got = np.array([L.oracle_fp16_to_fp32(int(b)) for b in all_bits], dtype=np.float32)
    finite = np.isfinite(ref)
    assert np.array_equal(got[finite].view(np.uint32), ref[finite].view(np.uint32))
    assert np.isnan(got[~finite]).sum() == np.isnan(ref[~finite]).sum()
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(2000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 300.0, 7e4)])
    want = vals.astype(np.float16).view(np.uint16)
    got16 = np.array([L.oracle_fp32_to_fp16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got16, want)


def test_bf16_rounding():
    L = oracle.lib()
    rng = np.random.default_rng(1)
    vals = rng.standard_normal(4000).astype(np.float32) * 3
    got = np.array([L.oracle_bf16_to_fp32(L.oracle_fp32_to_bf16(float(v))) for v in vals], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), oracle.fp32_to_bf16_round(vals).view(np.uint32))
    import torch
    want = torch.from_numpy(vals).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_matmul_reference_known_answers():
    # tests/InterpreterTest.cpp:50-96: [[1,2,3],[4,5,6]] @ [[1,2],[3,4],[5,6]] = [[22,28],[49,64]]
    x = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    wt = np.array([[1, 2], [3, 4], [5, 6]], dtype=np.float32)
    out = oracle.matmul_ikj(x, wt)
    assert out.tolist() == [[22, 28], [49, 64]]
    assert (out + np.array([[100, 200]], dtype=np.float32)).reshape(-1).tolist() == [122, 228, 149, 264]
    # tests/CUDADeviceTest.cpp:108-125: A @ A^T
    assert oracle.matmul_ikj(x, oracle.transpose(x)).tolist() == [[14, 32], [32, 77]]


def test_matmul_variants_are_bit_identical():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 640)).astype(np.float32)
    w = rng.standard_normal((70, 640)).astype(np.float32)
    ref = oracle.matmul_ikj(x, oracle.transpose(w))
    assert_bit_exact(oracle.matmul_nk(x, w, threads=1), ref, "nk 1 thread")
    assert_bit_exact(oracle.matmul_nk(x, w, threads=4), ref, "nk 4 threads")
    assert_bit_exact(oracle.matmul_ikj(x, oracle.transpose(w), threads=3), ref, "ikj 3 threads")
    assert np.allclose(ref, oracle.matmul_nk_f64(x, w), rtol=0, atol=1e-3)


def test_dequant_rejects_bad_shapes():
    # LLaMABuilder.cpp:121-126, 137-142
    with pytest.raises(ValueError):
        oracle.dequant(synth.Q4_0, np.zeros(18, dtype=np.uint8), 1, 48)
    with pytest.raises(ValueError):
        oracle.dequant(synth.Q4_0, np.zeros(17, dtype=np.uint8), 1, 32)
    with pytest.raises(ValueError):
        oracle.dequant(6, np.zeros(36, dtype=np.uint8), 1, 32)   # Q8_1 is not a tensor format of the importer


CARRIED = {"q4_1": 2, "q5_0": 3, "q5_1": 4, "q2_k": 7, "q3_k": 8, "q5_k": 10}


@pytest.mark.parametrize("name", sorted(CARRIED))
def test_carried_formats_golden_vectors(name):
    """The block formats the importer carries but nothing multiplies (tools/gguf/GGUFImporter.cpp:257-304):
    the oracle's dequantizers are bit-exact with the ggml project's Python ones on committed random payloads
    (tests/golden/dequant_carried_golden.npz, written by make_golden.py)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dequant_carried_golden.npz"))
    assert int(g[name + "_format"]) == CARRIED[name]
    n, k = int(g["rows"]), int(g["k"])
    got = oracle.dequant(CARRIED[name], g[name + "_payload"], n, k)
    assert_bit_exact(got, g[name + "_values"], name)

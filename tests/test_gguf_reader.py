"""The ggml-free GGUF reader (litenn_b200/host/GGUFReader.hpp) on the committed fixture
tests/golden/tiny_llama.gguf (written by tests/golden/make_gguf_fixture.py and cross-checked there
against the ggml project's own Python reader).  What is asserted follows the reference's importer
test (tests/GGUFImporterTest.cpp:469-535): metadata values, tensor names, reversed shapes, block
formats, byte counts and the first and last byte of the 18-byte Q4_0 payload."""
import importlib.util
import os
import subprocess

import numpy as np
import pytest

import oracle
from litenn_b200 import capi, synth

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "native", "gguf_reader_test.cpp")
EXE = os.path.join(HERE, "native", "gguf_reader_test")
FIXTURE = os.path.join(HERE, "golden", "tiny_llama.gguf")

spec = importlib.util.spec_from_file_location("make_gguf_fixture", os.path.join(HERE, "golden", "make_gguf_fixture.py"))
fixture = importlib.util.module_from_spec(spec)
spec.loader.exec_module(fixture)


@pytest.fixture(scope="module")
def reader_exe(qmm_lib):
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    deps = [SRC, os.path.join(ROOT, "litenn_b200", "host", "GGUFReader.hpp"),
            os.path.join(ROOT, "litenn_b200", "host", "LiteNNQuantMatMul.hpp"), os.path.join(ROOT, "include", "litenn_qmm.h")]
    if not os.path.exists(EXE) or any(os.path.getmtime(d) > os.path.getmtime(EXE) for d in deps):
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(cuda, "include"), "-o", EXE, SRC,
                        "-L", os.path.join(ROOT, "litenn_b200"), "-lqmm_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
                        "-Wl,-rpath," + os.path.join(ROOT, "litenn_b200"), "-Wl,-rpath," + os.path.join(cuda, "lib64")],
                       check=True)
    return EXE


def run(exe, *args):
    return subprocess.run([exe, *args], capture_output=True, text=True)


def test_fixture_is_what_the_generator_writes():
    assert open(FIXTURE, "rb").read() == fixture.build()


def test_lists_metadata_tensors_and_hyperparameters(reader_exe):
    r = run(reader_exe, "list", FIXTURE)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    assert lines[0] == "version 3"
    meta = {l.split()[1]: l.split(" ", 2)[2] for l in lines if l.startswith("meta ")}
    assert meta["general.architecture"] == "str llama"
    assert meta["llama.attention.head_count_kv"] == "u64 2"
    assert meta["tokenizer.ggml.tokens"] == "array 3 <s> a b"
    assert meta["tokenizer.ggml.scores"] == "array 3 0 -1 -2.5"
    assert meta["fixture.flag"] == "bool 1"
    assert meta["fixture.big"] == f"u64 {2 ** 40 + 5}"
    tensors = [l.split() for l in lines if l.startswith("tensor ")]
    want = fixture.tensors()
    assert [t[1] for t in tensors] == [w[0] for w in want]
    fmt_of = {fixture.T_F32: -1, fixture.T_Q4_0: 1, fixture.T_Q8_0: 5, fixture.T_Q4_K: 9, fixture.T_Q5_K: 10, fixture.T_Q6_K: 11}
    for t, (name, shape, ttype, payload) in zip(tensors, want):
        assert int(t[3]) == ttype and int(t[5]) == fmt_of[ttype] and int(t[7]) == len(payload)
        i = t.index("shape")
        assert tuple(int(x) for x in t[i + 1:t.index("first")]) == tuple(shape)      # outermost dimension first
        assert int(t[t.index("first") + 1]) == payload[0] and int(t[t.index("last") + 1]) == payload[-1]
    # the reference's 18-byte payload: [0] = 0x10, [17] = 0x7f, 18 bytes, expressed shape {32}
    q = [t for t in tensors if t[1] == "quantized.weight"][0]
    assert (int(q[7]), q[q.index("shape") + 1], int(q[q.index("first") + 1]), int(q[q.index("last") + 1])) == (18, "32", 0x10, 0x7F)
    h = [l for l in lines if l.startswith("hparams ")][0].split()
    assert h[1:11] == ["llama", "128", "64", "1", "256", "4", "2", "16", "2", "8"]
    assert float(h[11]) == 10000.0 and abs(float(h[12]) - 1e-5) < 1e-9


def test_payloads_are_byte_exact(reader_exe, tmp_path):
    for name, shape, ttype, payload in fixture.tensors():
        out = tmp_path / "p.bin"
        r = run(reader_exe, "payload", FIXTURE, name, str(out))
        assert r.returncode == 0, r.stdout
        assert out.read_bytes() == payload, name


def test_errors_are_runtime_errors_with_the_importers_wording(reader_exe, tmp_path):
    r = run(reader_exe, "list", str(tmp_path / "missing.gguf"))
    assert r.returncode == 3 and "Failed to open GGUF file" in r.stdout
    blob = fixture.build()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(blob[:len(blob) - 4000])          # the last tensors lose their bytes
    r = run(reader_exe, "list", str(cut))
    assert r.returncode == 3 and "inconsistent byte size" in r.stdout
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + blob[4:])
    r = run(reader_exe, "list", str(bad))
    assert r.returncode == 3 and "not a GGUF file" in r.stdout
    r = run(reader_exe, "payload", FIXTURE, "no.such.tensor", str(tmp_path / "x"))
    assert r.returncode == 3 and "has no tensor" in r.stdout


def test_container_variants_and_malformed_headers(reader_exe, tmp_path):
    """Version 2 has the same layout as version 3; an unknown version, an alignment that is not a power of two
    and an alignment the stored offsets do not honour are refused."""
    import struct
    blob = bytearray(fixture.build())
    v2 = tmp_path / "v2.gguf"
    v2.write_bytes(bytes(blob[:4]) + struct.pack("<I", 2) + bytes(blob[8:]))
    r = run(reader_exe, "list", str(v2))
    assert r.returncode == 0 and r.stdout.splitlines()[0] == "version 2"
    assert [l for l in r.stdout.splitlines() if l.startswith("tensor ")] == \
        [l for l in run(reader_exe, "list", FIXTURE).stdout.splitlines() if l.startswith("tensor ")]
    v9 = tmp_path / "v9.gguf"
    v9.write_bytes(bytes(blob[:4]) + struct.pack("<I", 9) + bytes(blob[8:]))
    r = run(reader_exe, "list", str(v9))
    assert r.returncode == 3 and "Unsupported GGUF version 9" in r.stdout
    key = b"general.alignment"
    at = blob.find(key) + len(key) + 4            # after the key: value type (u32), then the value
    assert struct.unpack_from("<I", blob, at)[0] == fixture.ALIGN
    odd = bytearray(blob)
    struct.pack_into("<I", odd, at, 24)
    bad = tmp_path / "odd_alignment.gguf"
    bad.write_bytes(bytes(odd))
    r = run(reader_exe, "list", str(bad))
    assert r.returncode == 3 and "power of two" in r.stdout
    wide = bytearray(blob)
    struct.pack_into("<I", wide, at, 4 * fixture.ALIGN)   # the stored offsets are multiples of ALIGN only
    bad = tmp_path / "wide_alignment.gguf"
    bad.write_bytes(bytes(wide))
    r = run(reader_exe, "list", str(bad))
    assert r.returncode == 3 and ("not aligned" in r.stdout or "inconsistent byte size" in r.stdout)


@pytest.mark.gpu
@pytest.mark.parametrize("name,fmt", [("blk.0.attn_q.weight", synth.Q4_0), ("token_embd.weight", synth.Q8_0),
                                      ("blk.0.ffn_up.weight", synth.Q4_K), ("blk.0.ffn_down.weight", synth.Q6_K)])
def test_file_to_packed_weight_dequantizes_bit_exactly(reader_exe, tmp_path, name, fmt):
    """File -> payload -> upload-time repack on the GPU -> dequantize: the oracle's values, bit for bit."""
    out = tmp_path / "w.bin"
    r = run(reader_exe, "pack", FIXTURE, name, str(out))
    assert r.returncode == 0, r.stdout + r.stderr
    shape, payload = [(s, p) for n, s, t, p in fixture.tensors() if n == name][0]
    want = oracle.dequant(fmt, np.frombuffer(payload, dtype=np.uint8), shape[0], shape[1])
    got = np.fromfile(out, dtype=np.float32).reshape(shape)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.gpu
def test_format_without_matmul_kernels_is_dequantized_on_the_device(reader_exe, tmp_path):
    """The fixture's Q5_K tensor: file -> raw payload on the GPU -> fp32, the oracle's values bit for bit."""
    out = tmp_path / "w.bin"
    r = run(reader_exe, "dequant", FIXTURE, "blk.0.ffn_gate.weight", str(out))
    assert r.returncode == 0, r.stdout + r.stderr
    shape, payload = [(s, p) for n, s, t, p in fixture.tensors() if n == "blk.0.ffn_gate.weight"][0]
    want = oracle.dequant(10, np.frombuffer(payload, dtype=np.uint8), shape[0], shape[1])
    got = np.fromfile(out, dtype=np.float32).reshape(shape)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.gpu
def test_formats_the_kernels_do_not_take_are_refused_not_misread(reader_exe, tmp_path):
    r = run(reader_exe, "pack", FIXTURE, "blk.0.ffn_gate.weight", str(tmp_path / "w.bin"))   # Q5_K: carried, not multiplied
    assert r.returncode == 3 and "block format 10" in r.stdout

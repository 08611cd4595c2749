"""Writes tests/golden/tiny_llama.gguf, a GGUF v3 archive of a tiny LLaMA-shaped model.

The container layout is the published one (magic, version, counts, metadata key/values,
tensor directory, aligned data section).  The tensors mirror what the reference's importer
test builds with ggml (tests/GGUFImporterTest.cpp:146-186, 298-341): a few `llama.*`
hyperparameters, an F32 norm, and block-quantized linears — among them the reference's own
18-byte Q4_0 payload `10 00 22 44 ... ff 7f` (GGUFImporterTest.cpp:173-176).  Payloads of the
quantized linears come from the same seeded generator the GPU tests use (litenn_b200.synth).

Run from the repository root:  python tests/golden/make_gguf_fixture.py
When the `gguf` Python package of the ggml project is importable, the script re-reads the
file with it and checks names, shapes, types and bytes, so the fixture is pinned to that reader.
"""
import os
import struct
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from litenn_b200 import synth  # noqa: E402

OUT = os.path.join(ROOT, "tests", "golden", "tiny_llama.gguf")
ALIGN = 32
T_F32, T_Q4_0, T_Q8_0, T_Q4_K, T_Q6_K, T_Q5_K = 0, 2, 8, 12, 14, 13
V_U32, V_F32, V_STR, V_ARR, V_U64, V_BOOL = 4, 6, 8, 9, 10, 7

REFERENCE_Q4_0 = bytes([0x10, 0x00, 0x22, 0x44, 0x66, 0x88, 0xaa, 0xcc, 0xee, 0x11, 0x33, 0x55, 0x77, 0x99, 0xbb,
                        0xdd, 0xff, 0x7f])


def gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def kv(key: str, vtype: int, payload: bytes) -> bytes:
    return gstr(key) + struct.pack("<I", vtype) + payload


def tensors():
    d, ffn, vocab = 64, 256, 64
    out = [
        ("token_embd.weight", (vocab, d), T_Q8_0, synth.make_weight(synth.Q8_0, vocab, d, seed=7, name="fx.embd").tobytes()),
        ("blk.0.attn_norm.weight", (d,), T_F32, synth.make_norm_weight(d, seed=7, name="fx.norm").tobytes()),
        ("blk.0.attn_q.weight", (d, d), T_Q4_0, synth.make_weight(synth.Q4_0, d, d, seed=7, name="fx.q").tobytes()),
        ("blk.0.ffn_down.weight", (d, ffn), T_Q6_K, synth.make_weight(synth.Q6_K, d, ffn, seed=7, name="fx.down").tobytes()),
        ("blk.0.ffn_up.weight", (ffn, 256), T_Q4_K, synth.make_weight(synth.Q4_K, ffn, 256, seed=7, name="fx.up").tobytes()),
        ("blk.0.ffn_gate.weight", (16, 256), T_Q5_K, bytes(range(176)) * 16),   # carried as a payload only
        ("quantized.weight", (32,), T_Q4_0, REFERENCE_Q4_0),
    ]
    return out


def build() -> bytes:
    meta = [
        kv("general.architecture", V_STR, gstr("llama")),
        kv("general.name", V_STR, gstr("tiny fixture")),
        kv("general.alignment", V_U32, struct.pack("<I", ALIGN)),
        kv("llama.context_length", V_U32, struct.pack("<I", 128)),
        kv("llama.embedding_length", V_U32, struct.pack("<I", 64)),
        kv("llama.block_count", V_U32, struct.pack("<I", 1)),
        kv("llama.feed_forward_length", V_U32, struct.pack("<I", 256)),
        kv("llama.attention.head_count", V_U32, struct.pack("<I", 4)),
        kv("llama.attention.head_count_kv", V_U32, struct.pack("<I", 2)),
        kv("llama.attention.layer_norm_rms_epsilon", V_F32, struct.pack("<f", 1e-5)),
        kv("llama.rope.freq_base", V_F32, struct.pack("<f", 10000.0)),
        kv("llama.rope.dimension_count", V_U32, struct.pack("<I", 8)),
        kv("tokenizer.ggml.tokens", V_ARR, struct.pack("<IQ", V_STR, 3) + gstr("<s>") + gstr("a") + gstr("b")),
        kv("tokenizer.ggml.scores", V_ARR, struct.pack("<IQ", V_F32, 3) + struct.pack("<3f", 0.0, -1.0, -2.5)),
        kv("fixture.flag", V_BOOL, b"\x01"),
        kv("fixture.big", V_U64, struct.pack("<Q", 2 ** 40 + 5)),
    ]
    ts = tensors()
    directory, data, offset = b"", b"", 0
    for name, shape, ttype, payload in ts:
        ne = tuple(reversed(shape))  # ggml keeps the innermost dimension first
        directory += gstr(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", n) for n in ne)
        directory += struct.pack("<IQ", ttype, offset)
        padded = payload + b"\0" * ((-len(payload)) % ALIGN)
        data += padded
        offset += len(padded)
    head = b"GGUF" + struct.pack("<IQQ", 3, len(ts), len(meta)) + b"".join(meta) + directory
    head += b"\0" * ((-len(head)) % ALIGN)
    return head + data


def check_with_gguf_package(path):
    try:
        import gguf
    except Exception:
        print("gguf package not importable: fixture written without the cross-check")
        return
    r = gguf.GGUFReader(path)
    want = {name: (shape, ttype, payload) for name, shape, ttype, payload in tensors()}
    assert len(r.tensors) == len(want)
    for t in r.tensors:
        shape, ttype, payload = want[t.name]
        assert tuple(int(x) for x in reversed(t.shape)) == tuple(shape), (t.name, t.shape)
        assert int(t.tensor_type) == ttype, t.name
        assert bytes(np.asarray(t.data).tobytes()) == payload, t.name
    assert str(bytes(r.fields["general.architecture"].parts[-1]), "utf-8") == "llama"
    print(f"cross-checked {len(want)} tensors with gguf {getattr(gguf, '__version__', '')}")


if __name__ == "__main__":
    blob = build()
    with open(OUT, "wb") as f:
        f.write(blob)
    print(f"wrote {OUT} ({len(blob)} bytes)")
    check_with_gguf_package(OUT)

"""Generate the committed golden fixtures for the block dequantizers.

Run in a container that has the `gguf` Python package (the ggml project's own
Python restatement of the block formats).  It draws random payloads, covering
every bit of every field (uniform random bytes, with the fp16 scale fields kept
finite), dequantizes them with `gguf.quants.dequantize`, and stores payload and
expected fp32 values.  The tests then compare the C oracle, and on a GPU the
CUDA path, with these files bit for bit.

    python tests/golden/make_golden.py                   # both files
    python tests/golden/make_golden.py --carried-only    # only dequant_carried_golden.npz
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from litenn_b200 import synth  # noqa: E402

ROWS, K = 24, 512  # 24 rows: not a multiple of 16, exercises row padding in the repack


def finite_fp16(payload2d, col):
    """Clear the exponent's top bit of the fp16 at byte `col` so it is finite and modest."""
    payload2d[:, col + 1] &= 0xBF


def main():
    import gguf
    from gguf import quants

    types = {
        synth.Q4_0: gguf.GGMLQuantizationType.Q4_0,
        synth.Q8_0: gguf.GGMLQuantizationType.Q8_0,
        synth.Q4_K: gguf.GGMLQuantizationType.Q4_K,
        synth.Q6_K: gguf.GGMLQuantizationType.Q6_K,
    }
    out = {}
    for fmt, gt in types.items():
        name = synth.FORMAT_NAMES[fmt]
        rng = synth.rng_for(1234, "golden-" + name)
        nblk = ROWS * (K // synth.BLOCK_ELEMS[fmt])
        raw = rng.integers(0, 256, size=(nblk, synth.BLOCK_BYTES[fmt]), dtype=np.uint8)
        if fmt in (synth.Q4_0, synth.Q8_0):
            finite_fp16(raw, 0)
        elif fmt == synth.Q4_K:
            finite_fp16(raw, 0)
            finite_fp16(raw, 2)
        else:
            finite_fp16(raw, 208)
        rows = raw.reshape(ROWS, -1)
        deq = quants.dequantize(rows, gt).astype(np.float32).reshape(ROWS, K)
        out[name + "_payload"] = raw.reshape(-1)
        out[name + "_values"] = deq
        # the synthetic distribution used by the benchmark configs as well
        syn = synth.make_weight(fmt, ROWS, K, seed=7, name="golden-syn-" + name)
        out[name + "_syn_payload"] = syn
        out[name + "_syn_values"] = quants.dequantize(syn.reshape(ROWS, -1), gt).astype(np.float32).reshape(ROWS, K)
    out["rows"] = np.int64(ROWS)
    out["k"] = np.int64(K)
    np.savez_compressed(os.path.join(HERE, "dequant_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "dequant_golden.npz"))


# Formats the importer carries as payloads and this library only dequantizes: name -> (LiteNN
# QuantizedBlockFormat value, elements per block, bytes per block, byte offsets of the fp16 fields).
CARRIED = {
    "q4_1": (2, 32, 20, (0, 2)),
    "q5_0": (3, 32, 22, (0,)),
    "q5_1": (4, 32, 24, (0, 2)),
    "q2_k": (7, 256, 84, (80, 82)),
    "q3_k": (8, 256, 110, (108,)),
    "q5_k": (10, 256, 176, (0, 2)),
}


def main_carried():
    import gguf
    from gguf import quants

    out = {}
    for name, (fmt, elems, nbytes, halves) in CARRIED.items():
        gt = getattr(gguf.GGMLQuantizationType, name.upper())
        rng = synth.rng_for(4321, "golden-carried-" + name)
        raw = rng.integers(0, 256, size=(ROWS * (K // elems), nbytes), dtype=np.uint8)
        for col in halves:
            finite_fp16(raw, col)
        deq = quants.dequantize(raw.reshape(ROWS, -1), gt).astype(np.float32).reshape(ROWS, K)
        out[name + "_payload"] = raw.reshape(-1)
        out[name + "_values"] = deq
        out[name + "_format"] = np.int64(fmt)
    out["rows"] = np.int64(ROWS)
    out["k"] = np.int64(K)
    np.savez_compressed(os.path.join(HERE, "dequant_carried_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "dequant_carried_golden.npz"))


if __name__ == "__main__":
    if "--carried-only" not in sys.argv:
        main()
    main_carried()

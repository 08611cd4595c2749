"""Shared pieces of the parity tests."""
import numpy as np

from litenn_b200 import synth

FORMATS = [synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K]

# Matmul parity bar: max |a - e| <= REL_TOL * max|e| over the output tensor
# (max relative error 1e-3 with fp32 accumulation; normalising by the largest
# expected magnitude keeps outputs that cancel to ~0 from dividing by ~0).
REL_TOL = 1e-3


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_exact(actual, expected, what=""):
    a, e = bits(actual), bits(expected)
    if not np.array_equal(a, e):
        bad = np.flatnonzero(a.reshape(-1) != e.reshape(-1))
        i = int(bad[0])
        raise AssertionError(
            f"{what}: {bad.size} of {a.size} values differ; first at flat index {i}: "
            f"got {actual.reshape(-1)[i]!r} expected {expected.reshape(-1)[i]!r}")


def max_rel_err(actual, expected):
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    scale = np.abs(expected).max()
    if scale == 0.0:
        return float(np.abs(actual).max())
    return float(np.abs(actual - expected).max() / scale)


def random_payload(fmt, n, k, seed):
    """Uniform random bytes in every field (all nibble/6-bit/scale patterns), fp16 scales kept finite."""
    rng = np.random.default_rng(seed)
    p = rng.integers(0, 256, size=(n * (k // synth.BLOCK_ELEMS[fmt]), synth.BLOCK_BYTES[fmt]), dtype=np.uint8)
    for col in {synth.Q4_0: [1], synth.Q8_0: [1], synth.Q4_K: [1, 3], synth.Q6_K: [209]}[fmt]:
        p[:, col] &= 0xBF
    return p.reshape(-1)

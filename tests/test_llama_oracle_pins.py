"""Pins the decoder oracle's building blocks (oracle/llama_ref.py) to the known answers that the
reference's own layer tests hold (tests/LayerTest.cpp): inputs, expected values and tolerances are
the ones of the cited TEST bodies; where the reference computes its expectation with a helper of
its test file, the expectation here is recomputed with plain scalar loops, independent of the
oracle's vectorised code."""
import math

import numpy as np

from oracle import llama_ref as R


def near(a, e, tol):
    assert abs(float(a) - float(e)) <= tol, (a, e, tol)


# ---- RMSNorm (tests/LayerTest.cpp:1200-1264) --------------------------------------------------------

def test_rmsnorm_output_mean_square_near_one():
    out = R.rmsnorm(np.array([[1.0, 2.0, 3.0, 4.0]], np.float32), np.ones(4, np.float32), 1e-6)
    near(float((out.astype(np.float32) ** 2).mean()), 1.0, 1e-4)


def test_rmsnorm_zero_input_stays_zero():
    out = R.rmsnorm(np.zeros((1, 3), np.float32), np.ones(3, np.float32), 1e-6)
    for v in out.reshape(-1):
        near(v, 0.0, 1e-6)


def test_rmsnorm_weight_scales_normalized_output():
    out = R.rmsnorm(np.array([[1.0, 2.0, 3.0]], np.float32), np.full(3, 2.0, np.float32), 1e-6).reshape(-1)
    denom = np.sqrt(np.float32((1.0 + 4.0 + 9.0) / 3.0 + 1e-6))
    for i, x in enumerate((1.0, 2.0, 3.0)):
        near(out[i], 2.0 * x / denom, 1e-5)


def test_rmsnorm_scale_is_applied_in_double_before_the_single_cast():
    # src/LiteNN/ComputePrimitives.h:755-816: dst = (T)(x / denom * w) with every factor a double.
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 64)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(64)).astype(np.float32)
    want = np.empty_like(x)
    for r in range(3):
        var = sum(float(v) * float(v) for v in x[r]) / 64.0
        denom = math.sqrt(var + 1e-6)
        for i in range(64):
            want[r, i] = np.float32(float(x[r, i]) / denom * float(w[i]))
    assert np.array_equal(R.rmsnorm(x, w, 1e-6).view(np.uint32), want.view(np.uint32))


# ---- RoPE (tests/LayerTest.cpp:1269-1324) -----------------------------------------------------------

def test_rope_position_zero_is_identity():
    cos, sin = R.rope_tables(1, 4, 10000.0)
    out = R.rope(np.array([[1.0, 2.0, 3.0, 4.0]], np.float32), cos, sin).reshape(-1)
    for a, e in zip(out, (1.0, 2.0, 3.0, 4.0)):
        near(a, e, 1e-5)


def test_rope_rotates_pairs_at_position_one():
    cos, sin = R.rope_tables(2, 4, 1.0)
    out = R.rope(np.array([[0, 0, 0, 0], [1, 0, 0, 1]], np.float32), cos, sin).reshape(-1)
    c1, s1 = math.cos(1.0), math.sin(1.0)
    near(out[4], c1, 1e-5)
    near(out[5], s1, 1e-5)
    near(out[6], -s1, 1e-5)
    near(out[7], c1, 1e-5)


def test_rope_applies_frequency_scale_and_offset():
    cos, sin = R.rope_tables(2, 2, 1.0, position_offset=1, frequency_scale=0.5)
    out = R.rope(np.array([[0, 0], [1, 0]], np.float32), cos, sin).reshape(-1)
    near(out[2], math.cos(1.0), 1e-5)
    near(out[3], math.sin(1.0), 1e-5)


def test_rope_partial_rotation_keeps_the_tail():
    # tools/gguf/LLaMABuilder.cpp:311-348: rope.dimension_count < head_dim rotates the prefix with
    # frequencies over that count and passes the rest through.
    import dataclasses
    from litenn_b200 import llama as ll, synth
    spec = ll.LlamaSpec(n_layers=1, d_model=64, n_heads=1, n_kv_heads=1, head_dim=64, ffn=64, vocab=32,
                        linear_fmt=synth.Q8_0, embd_fmt=synth.Q8_0, max_seq=8, max_prefill=4, rope_dim=32)
    o = R.LlamaOracle(spec)
    x = np.arange(2 * 64, dtype=np.float32).reshape(2, 64) / 64.0
    out = o._rope_heads(x, 1, np.array([0, 3]))
    assert np.array_equal(out[:, 32:], x[:, 32:])
    assert np.array_equal(out[0], x[0])
    cos, sin = R.rope_tables(4, 32, spec.rope_theta)
    assert np.array_equal(out[1, :32], R.rope(x[1:2, :32], cos[3:4], sin[3:4])[0])
    near(out[1, 2], x[1, 2] * math.cos(3.0 * 10000.0 ** (-2.0 / 32)) - x[1, 3] * math.sin(3.0 * 10000.0 ** (-2.0 / 32)), 1e-5)


# ---- SiLU / SwiGLU (tests/LayerTest.cpp:1326-1392) --------------------------------------------------

def test_silu_matches_analytic_value():
    near(R.silu(np.array([2.0], np.float32))[0], 2.0 / (1.0 + math.exp(-2.0)), 1e-5)


def test_swiglu_identity_projections():
    eye = np.eye(2, dtype=np.float32)
    out = R.swiglu(np.array([[1.0, 2.0]], np.float32), eye, eye, eye).reshape(-1)
    near(out[0], 1.0 * (1.0 / (1.0 + math.exp(-1.0))) * 1.0, 1e-5)
    near(out[1], 2.0 * (1.0 / (1.0 + math.exp(-2.0))) * 2.0, 1e-5)


def test_swiglu_down_projection_changes_width():
    eye = np.eye(2, dtype=np.float32)
    out = R.swiglu(np.array([[1.0, 2.0]], np.float32), eye, eye, np.ones((2, 1), np.float32))
    assert out.shape == (1, 1)
    e0 = 1.0 * (1.0 / (1.0 + math.exp(-1.0))) * 1.0
    e1 = 2.0 * (1.0 / (1.0 + math.exp(-2.0))) * 2.0
    near(out[0, 0], e0 + e1, 1e-5)


# ---- attention (tests/LayerTest.cpp:304-440) --------------------------------------------------------

def scalar_attention(q, k, v, scale, query_offset=0):
    out = []
    for i, qi in enumerate(q):
        scores = []
        for j, kj in enumerate(k):
            s = sum(a * b for a, b in zip(qi, kj)) * scale
            if j > i + query_offset:
                s += -1.0e9
            scores.append(s)
        mx = max(scores)
        e = [math.exp(s - mx) for s in scores]
        z = sum(e)
        out.append([sum(e[j] / z * v[j][c] for j in range(len(k))) for c in range(len(v[0]))])
    return out


def test_attention_applies_causal_mask_before_softmax():
    q = [[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]
    k = [[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]
    v = [[2.0], [5.0], [11.0]]
    got = R.attention(np.array(q, np.float32), np.array(k, np.float32), np.array(v, np.float32), 1.0 / math.sqrt(2.0))
    want = scalar_attention(q, k, v, 1.0 / math.sqrt(2.0))
    for a, e in zip(got.reshape(-1), np.array(want).reshape(-1)):
        near(a, e, 1e-5)
    near(got[0, 0], 2.0, 1e-5)  # the first query sees only the first key


def test_attention_rectangular_causal_decode_mask():
    q, k, v = [[1.0, 0.0]], [[1.0, 0.0], [0.0, 1.0], [10.0, 0.0]], [[2.0], [5.0], [1000.0]]
    got = R.attention(np.array(q, np.float32), np.array(k, np.float32), np.array(v, np.float32), 1.0, query_offset=1)
    near(got[0, 0], scalar_attention(q, k, v, 1.0, query_offset=1)[0][0], 1e-5)
    assert got[0, 0] < 5.0  # the third key (value 1000) is in the future of a query at position 1


# ---- KV cache (tests/LayerTest.cpp:1449-1515) -------------------------------------------------------

def test_kv_append_concatenates_past_and_present():
    keys = R.kv_append(np.array([[1, 2], [3, 4]], np.float32), np.array([[5, 6]], np.float32)).reshape(-1)
    vals = R.kv_append(np.array([[10, 11, 12], [13, 14, 15]], np.float32), np.array([[16, 17, 18]], np.float32)).reshape(-1)
    assert keys.size == 6 and vals.size == 9
    near(keys[0], 1.0, 1e-5)
    near(keys[4], 5.0, 1e-5)
    near(keys[5], 6.0, 1e-5)
    near(vals[6], 16.0, 1e-5)
    near(vals[8], 18.0, 1e-5)


def test_decode_step_by_step_equals_one_longer_prefill_in_the_oracle():
    # the property tests/GGUFImporterTest.cpp:880-908 checks on the reference: feeding tokens one by one
    # with the explicit KV cache gives the logits of processing them at once (fp32 path on both sides)
    from litenn_b200 import llama as ll, synth
    spec = ll.LlamaSpec(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn=96, vocab=64,
                        linear_fmt=synth.Q8_0, embd_fmt=synth.Q8_0, max_seq=16, max_prefill=8, unit_norms=False,
                        rope_dim=8)
    toks = synth.make_token_ids(6, spec.vocab, seed=2, name="pin")
    a = R.LlamaOracle(spec, seed=1)
    a._forward(list(toks), False)
    b = R.LlamaOracle(spec, seed=1)
    for t in toks:
        b.decode_step(int(t))
    # the fp16 K/V cache is written identically on both sides, so only accumulation order differs
    assert np.abs(a.last_logits - b.last_logits).max() <= 1e-5 * np.abs(a.last_logits).max()

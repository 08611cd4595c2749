"""Decoder harness on the GPU against the numpy oracle: logits and greedy tokens.

Model sizes are small enough for the CPU oracle; the full 7B shape is exercised for
determinism and for "prefill then decode equals a longer prefill" (the property the
reference tests in tests/GGUFImporterTest.cpp:880-908).
"""
import numpy as np
import pytest

from litenn_b200 import capi, synth
from litenn_b200 import llama as ll

pytestmark = pytest.mark.gpu

SMALL_Q4_0 = ll.LlamaSpec(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                          linear_fmt=synth.Q4_0, embd_fmt=synth.Q6_K, max_seq=64, max_prefill=32)
SMALL_K = ll.LlamaSpec(n_layers=3, d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=768, vocab=1024,
                       linear_fmt=synth.Q4_K, down_fmt=synth.Q6_K, embd_fmt=synth.Q6_K, max_seq=64, max_prefill=32)


@pytest.fixture(scope="module")
def stream(qmm_lib):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    s = torch.cuda.Stream()
    yield s.cuda_stream
    del s


def rel_err(a, e):
    return float(np.abs(a - e).max() / np.abs(e).max())


MODES = [capi.LL_DECODE_GRAPH, capi.LL_DECODE_PERSISTENT]
MODE_IDS = ["graph", "persistent"]


@pytest.mark.parametrize("mode", MODES, ids=MODE_IDS)
@pytest.mark.parametrize("spec", [SMALL_Q4_0, SMALL_K], ids=["q4_0", "q4_k+q6_k"])
def test_prefill_and_greedy_decode_match_oracle(stream, spec, mode):
    from oracle.llama_ref import LlamaOracle
    prompt = synth.make_token_ids(20, spec.vocab, seed=5, name="prompt")
    steps = 16
    ref = LlamaOracle(spec, seed=0)
    model = ll.LlamaModel(spec, stream=stream, seed=0)
    model.set_decode_mode(mode)
    tok_ref = ref.prefill(prompt)
    tok = model.prefill(prompt)
    # prefill rounds activations and weights to bf16 on both sides; what is left is fp32 vs fp64 accumulation
    assert rel_err(model.last_logits(), ref.last_logits) <= 1e-2
    gaps = [ref.top2_gap()]
    ref_tokens, cur = [tok_ref], tok_ref
    for _ in range(steps):
        cur = ref.decode_step(cur)
        ref_tokens.append(cur)
        gaps.append(ref.top2_gap())
    got_tokens = [tok] + model.decode(steps).tolist()
    assert capi.kernel_status(0) == 0
    for i, (a, e) in enumerate(zip(got_tokens, ref_tokens)):
        if a != e:
            gap, scale = gaps[i]
            # a flip is only excusable when the oracle's own top-2 logits are closer than the matmul bar
            assert gap <= 1e-3 * scale, f"token {i}: got {a}, oracle {e}, top-2 gap {gap:.3e} of {scale:.3e}"
            pytest.skip(f"sequences part at step {i} on a near-tie (gap {gap:.2e})")
    assert got_tokens == ref_tokens


@pytest.mark.parametrize("mode", MODES, ids=MODE_IDS)
def test_decode_logits_match_oracle(stream, mode):
    from oracle.llama_ref import LlamaOracle
    spec = SMALL_Q4_0
    prompt = synth.make_token_ids(9, spec.vocab, seed=6, name="prompt2")
    ref = LlamaOracle(spec, seed=0)
    model = ll.LlamaModel(spec, stream=stream, seed=0)
    model.set_decode_mode(mode)
    t_ref, t = ref.prefill(prompt), model.prefill(prompt)
    for _ in range(3):
        # feed the oracle's token to both so that one flip cannot hide later errors
        t_ref = ref.decode_step(t_ref)
    got = model.decode(3)
    # decode keeps fp32 activations and exact weights: only the 16-bit activation quantization differs
    assert rel_err(model.last_logits(), ref.last_logits) <= 5e-3
    assert got[-1] == t_ref or ref.top2_gap()[0] <= 1e-3 * ref.top2_gap()[1]


@pytest.mark.parametrize("mode", MODES, ids=MODE_IDS)
def test_decode_is_deterministic_and_resettable(stream, mode):
    spec = SMALL_K
    prompt = synth.make_token_ids(12, spec.vocab, seed=7, name="prompt3")
    model = ll.LlamaModel(spec, stream=stream, seed=1)
    model.set_decode_mode(mode)
    first = [model.prefill(prompt)] + model.decode(10).tolist()
    model.reset()
    second = [model.prefill(prompt)] + model.decode(10).tolist()
    assert first == second


def test_invalid_calls_are_rejected(stream):
    spec = SMALL_Q4_0
    model = ll.LlamaModel(spec, stream=stream, seed=0)
    with pytest.raises(capi.QmmError):
        model.prefill(np.zeros(spec.max_prefill + 1, dtype=np.int32))
    model.prefill(synth.make_token_ids(8, spec.vocab, seed=1, name="p"))
    with pytest.raises(capi.QmmError):
        model.decode(spec.max_seq)  # beyond the KV cache


def test_both_decode_modes_agree_on_the_7b_shape(stream):
    """Four blocks of the 7B shape (too large for the CPU oracle): the per-operator graph and the
    persistent kernel must pick the same tokens; their logits differ only by fp32 summation order."""
    import dataclasses
    spec = dataclasses.replace(ll.SPEC_7B, n_layers=4)
    prompt = synth.make_token_ids(64, spec.vocab, seed=3, name="prompt7b")
    out, logits = [], []
    for mode in MODES:
        model = ll.LlamaModel(spec, stream=stream, seed=0, share_layer_payloads=True)
        model.set_decode_mode(mode)
        first = model.prefill(prompt)
        out.append([first] + model.decode(12).tolist())
        logits.append(model.last_logits())
        model.close()
    assert rel_err(logits[1], logits[0]) <= 1e-3
    assert out[0] == out[1]


def test_persistent_mode_is_refused_for_tensor_parallel_shards(stream):
    spec = SMALL_Q4_0
    model = ll.LlamaModel(spec, stream=stream, seed=0, tp_rank=0, tp_size=2)
    model.set_decode_mode(capi.LL_DECODE_PERSISTENT)
    with pytest.raises(capi.QmmError):
        model.decode(1)

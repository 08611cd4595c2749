"""Decoder harness on the GPU against the numpy oracle: logits and greedy tokens.

Small models cover every format and option; the benchmark configurations are compared with
the oracle at their own dimensions (d_model, heads, head_dim, FFN width, formats, prompt
length) with few blocks, so that the CPU side stays tractable.
"""
import dataclasses

import numpy as np
import pytest

from litenn_b200 import capi, synth
from litenn_b200 import llama as ll

pytestmark = pytest.mark.gpu

SMALL_Q4_0 = ll.LlamaSpec(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                          linear_fmt=synth.Q4_0, embd_fmt=synth.Q6_K, max_seq=64, max_prefill=32)
SMALL_K = ll.LlamaSpec(n_layers=3, d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=768, vocab=1024,
                       linear_fmt=synth.Q4_K, down_fmt=synth.Q6_K, embd_fmt=synth.Q6_K, max_seq=64, max_prefill=32)
# trained-model features the benchmark configurations do not have: norm weights other than one,
# a rotary dimension below the head dimension, logits from the embedding matrix
SMALL_OPTS = ll.LlamaSpec(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, head_dim=128, ffn=512, vocab=512,
                          linear_fmt=synth.Q8_0, embd_fmt=synth.Q6_K, max_seq=64, max_prefill=32,
                          rope_dim=64, unit_norms=False, tied_output=True)


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


def compare_with_oracle(stream, spec, prompt, steps, share=False, prefill_tol=1e-2, decode_tol=5e-3):
    """Prefill + greedy decode on both sides; logits after the prefill and after the last step; tokens
    identical unless the oracle's own top-2 logits are closer than the matmul bar."""
    from oracle.llama_ref import LlamaOracle
    ref = LlamaOracle(spec, seed=0, share_layer_payloads=share)
    model = ll.LlamaModel(spec, stream=stream, seed=0, share_layer_payloads=share)
    tok_ref = ref.prefill(prompt)
    tok = model.prefill(prompt)
    # prefill rounds activations and weights to bf16 on both sides; what is left is fp32 vs fp64 accumulation
    err_prefill = rel_err(model.last_logits(), ref.last_logits)
    assert err_prefill <= prefill_tol, err_prefill
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
    # decode keeps fp32 activations and exact weights: only the 16-bit activation quantization differs
    err_decode = rel_err(model.last_logits(), ref.last_logits)
    assert err_decode <= decode_tol, err_decode
    model.close()
    return err_prefill, err_decode


@pytest.mark.parametrize("spec", [SMALL_Q4_0, SMALL_K, SMALL_OPTS], ids=["q4_0", "q4_k+q6_k", "q8_0+norms+partial-rope+tied"])
def test_prefill_and_greedy_decode_match_oracle(stream, spec):
    prompt = synth.make_token_ids(20, spec.vocab, seed=5, name="prompt")
    compare_with_oracle(stream, spec, prompt, 16)


def test_decode_from_an_empty_cache_matches_oracle(stream):
    """No prefill at all: position 0 onwards through the decode path (fp32 on both sides)."""
    from oracle.llama_ref import LlamaOracle
    spec = SMALL_OPTS
    ref = LlamaOracle(spec, seed=0)
    model = ll.LlamaModel(spec, stream=stream, seed=0)
    cur = 7
    for i in range(5):
        want = ref.decode_step(cur)
        got = model.step_host(cur)
        assert rel_err(model.last_logits(), ref.last_logits) <= 5e-3
        assert got == want or ref.top2_gap()[0] <= 1e-3 * ref.top2_gap()[1]
        cur = want
    assert model.has_graph()  # single-step calls replay the graph from the second token on


def test_7b_shape_two_blocks_against_oracle(stream):
    """configs[3] at its own dimensions (d 4096, 32 heads x 128, FFN 11008, vocab 32000, Q4_0 + Q6_K),
    two blocks, the 512-token prompt through the tcgen05 prefill, then 16 greedy steps."""
    spec = dataclasses.replace(ll.SPEC_7B, n_layers=2, max_seq=544)
    prompt = synth.make_token_ids(512, spec.vocab, seed=0, name="prompt")
    errs = compare_with_oracle(stream, spec, prompt, 16)
    print("7B-shape logits error after prefill / after decode:", errs)


def test_70b_shape_one_block_against_oracle(stream):
    """configs[4] at its own dimensions (d 8192, 64 query / 8 kv heads x 128, FFN 28672, Q4_K linears,
    Q6_K ffn_down and output), one block, the vocabulary cut to 8192 rows, a 64-token prompt."""
    spec = dataclasses.replace(ll.SPEC_70B, n_layers=1, vocab=8192, max_seq=96, max_prefill=64)
    prompt = synth.make_token_ids(64, spec.vocab, seed=0, name="prompt70")
    errs = compare_with_oracle(stream, spec, prompt, 8)
    print("70B-shape logits error after prefill / after decode:", errs)


def test_decode_is_deterministic_and_resettable(stream):
    spec = SMALL_K
    prompt = synth.make_token_ids(12, spec.vocab, seed=7, name="prompt3")
    model = ll.LlamaModel(spec, stream=stream, seed=1)
    first = [model.prefill(prompt)] + model.decode(10).tolist()
    model.reset()
    second = [model.prefill(prompt)] + model.decode(10).tolist()
    assert first == second


def test_eager_single_steps_equal_graph_replays(stream):
    """Tokens enqueued one call at a time without a synchronize in between (the first runs eagerly, the
    rest replay the graph) must equal one multi-step call: nothing may read the position early."""
    spec = SMALL_Q4_0
    prompt = synth.make_token_ids(10, spec.vocab, seed=8, name="prompt4")
    a = ll.LlamaModel(spec, stream=stream, seed=0)
    first = a.prefill(prompt)
    want = a.decode(12).tolist()
    b = ll.LlamaModel(spec, stream=stream, seed=0)
    assert b.prefill(prompt) == first
    for _ in range(12):
        b.decode_enqueue(1)
    got = b.decode(1).tolist()        # synchronizes; the 13th token
    a_next = a.decode(1).tolist()
    assert got == a_next
    assert b.has_graph()


def test_invalid_calls_are_rejected(stream):
    spec = SMALL_Q4_0
    model = ll.LlamaModel(spec, stream=stream, seed=0)
    with pytest.raises(capi.QmmError):
        model.prefill(np.zeros(spec.max_prefill + 1, dtype=np.int32))
    model.prefill(synth.make_token_ids(8, spec.vocab, seed=1, name="p"))
    with pytest.raises(capi.QmmError):
        model.decode(spec.max_seq)  # beyond the KV cache
    with pytest.raises(capi.QmmError):
        ll.LlamaModel(dataclasses.replace(spec, ffn=520), stream=stream)  # FFN width not a multiple of 32


def test_a_peer_that_never_answers_is_reported_not_waited_for(stream):
    """Failure detection without a fault: a tensor-parallel rank whose peers' slots are never filled
    (loopback hook) gives up after the wait limit, reports QMM_E_KERNEL, and later steps do not wait
    again until the model is reset."""
    import time
    spec = dataclasses.replace(SMALL_Q4_0, n_layers=1)
    model = ll.LlamaModel(spec, stream=stream, seed=0, tp_rank=0, tp_size=2)
    model.tp_loopback()
    model.set_wait_limit(1 << 10)
    with pytest.raises(capi.QmmError) as e:
        model.decode(1)
    assert e.value.code == capi.E_KERNEL and "status 5" in str(e.value)
    t0 = time.perf_counter()
    with pytest.raises(capi.QmmError) as e:
        model.decode(4)
    assert e.value.code == capi.E_KERNEL
    assert time.perf_counter() - t0 < 5.0
    model.reset()                      # clears the status; the next step runs into the limit again
    with pytest.raises(capi.QmmError) as e:
        model.decode(1)
    assert e.value.code == capi.E_KERNEL
    model.close()
    assert capi.kernel_status(0) == 0  # the library's own status word was never involved


def batch_against_oracles(stream, spec, batch, prompt_lens, steps):
    """Batched decode: every sequence against its own run of the oracle (prompt lengths differ, so the
    sequences sit at different positions of their caches in every step)."""
    from oracle.llama_ref import LlamaOracle
    model = ll.LlamaModel(spec, stream=stream, seed=0)
    model.batch_create(batch, steps)
    want = np.zeros((steps, batch), dtype=np.int64)
    excused_from = [steps] * batch
    for b in range(batch):
        ref = LlamaOracle(spec, seed=0)
        prompt = synth.make_token_ids(prompt_lens[b], spec.vocab, seed=11 + b, name="batch-prompt")
        cur = ref.prefill(prompt)
        got_first = model.batch_prefill(b, prompt)
        gap, scale = ref.top2_gap()
        assert got_first == cur or gap <= 1e-3 * scale, (b, got_first, cur)
        cur = got_first                       # both sides continue from the same token
        for s in range(steps):
            cur = ref.decode_step(cur)
            want[s, b] = cur
            gap, scale = ref.top2_gap()
            if gap <= 1e-3 * scale:           # a near-tie: what follows may legitimately part
                excused_from[b] = min(excused_from[b], s)
    got = model.batch_decode(steps)
    assert capi.kernel_status(0) == 0
    assert got.shape == (steps, batch)
    for b in range(batch):
        upto = excused_from[b]
        assert got[:upto, b].tolist() == want[:upto, b].tolist(), f"sequence {b}"
    assert sum(excused_from) >= steps * batch * 0.8     # the excuse must stay the exception
    model.close()


@pytest.mark.parametrize("spec,batch", [(SMALL_Q4_0, 3), (SMALL_K, 16), (SMALL_OPTS, 5), (SMALL_Q4_0, 1)],
                         ids=["q4_0-b3", "q4_k+q6_k-b16", "q8_0+norms+partial-rope+tied-b5", "q4_0-b1"])
def test_batched_decode_matches_one_oracle_per_sequence(stream, spec, batch):
    lens = [4 + (5 * b) % 17 for b in range(batch)]
    batch_against_oracles(stream, spec, batch, lens, 10)


def test_batched_decode_70b_shape_one_block(stream):
    """configs[4] dimensions (GQA 64 / 8, Q4_K + Q6_K), one block, vocabulary cut to 8192 rows, batch 4."""
    spec = dataclasses.replace(ll.SPEC_70B, n_layers=1, vocab=8192, max_seq=64, max_prefill=32)
    batch_against_oracles(stream, spec, 4, [9, 16, 5, 12], 4)


def test_batched_decode_steps_add_up_and_limits_hold(stream):
    """Two calls of 3 and 4 steps give the 7 steps of one call; identical prompts give identical columns that
    equal the single-sequence decode; capacity errors are reported, not run into."""
    spec = SMALL_K
    prompt = synth.make_token_ids(9, spec.vocab, seed=3, name="same-prompt")
    single = ll.LlamaModel(spec, stream=stream, seed=0)
    first = single.prefill(prompt)
    alone = single.decode(7)
    single.close()
    model = ll.LlamaModel(spec, stream=stream, seed=0)
    with pytest.raises(capi.QmmError):
        model.batch_decode_enqueue(1)                     # no batch yet
    # the single sequence is in use (position 12) when the batch is set up, and goes on afterwards
    assert model.prefill(prompt) == first
    assert model.decode(3).tolist() == alone[:3].tolist()
    model.batch_create(4, 7)
    with pytest.raises(capi.QmmError):
        model.batch_create(2, 7)                          # one batch per model
    for b in range(4):
        assert model.batch_prefill(b, prompt) == first
    with pytest.raises(capi.QmmError):
        model.batch_prefill(1, prompt)                    # that sequence already holds a prompt
    a = model.batch_decode(3)
    c = model.batch_decode(4)
    both = np.concatenate([a, c])
    assert (both == both[:, :1]).all()
    assert both[:, 0].tolist() == alone.tolist()
    assert (model.batch_generated(0, 7) == both).all()
    with pytest.raises(capi.QmmError):
        model.batch_decode(1)                             # max_steps reached
    assert model.decode(4).tolist() == alone[3:].tolist()  # the single sequence was not disturbed
    model.reset()                                         # all sequences start over
    for b in range(4):
        assert model.batch_prefill(b, prompt) == first
    assert (model.batch_decode(7) == both).all()
    model.close()

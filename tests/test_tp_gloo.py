"""Tensor-parallel host logic on the CPU: two `gloo` ranks shard one decoder block with
`shard_ranges`, run their parts with the oracle's dequantized weights, exchange exactly where
the GPU path does (all-reduce after attention-out and FFN-down, gather of argmax candidates)
and must reproduce the unsharded block."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from litenn_b200 import llama as ll
from litenn_b200 import synth

SPEC = ll.LlamaSpec(n_layers=1, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                    linear_fmt=synth.Q4_0, embd_fmt=synth.Q6_K, max_seq=16, max_prefill=8)


def _block_parts(rank, world):
    s = SPEC
    p = ll.tensor_payloads(s, 0, seed=0)
    d, hd = s.d_model, s.head_dim
    w = {k: oracle.dequant(s.linear_fmt, p[k], n, kk) for k, (n, kk) in {
        "attn_q": (s.n_heads * hd, d), "attn_k": (s.n_kv_heads * hd, d), "attn_v": (s.n_kv_heads * hd, d),
        "attn_output": (d, s.n_heads * hd), "ffn_gate": (s.ffn, d), "ffn_up": (s.ffn, d), "ffn_down": (d, s.ffn)}.items()}
    if world == 1:
        return w
    out = {}
    for name, (kind, a, b) in ll.shard_ranges(s, rank, world).items():
        if name in w:
            out[name] = w[name][a:b] if kind == "rows" else w[name][:, a:b]
    return out


def _block(x, w, reduce):
    """One token at position 0 (attention over itself = v), sharded or not."""
    q, k, v = x @ w["attn_q"].T, x @ w["attn_k"].T, x @ w["attn_v"].T
    group = w["attn_q"].shape[0] // w["attn_k"].shape[0]
    ctx = np.repeat(v.reshape(-1, SPEC.head_dim), group, axis=0).reshape(-1)   # softmax over one key = 1
    h = x + reduce(ctx @ w["attn_output"].T)
    act = (h @ w["ffn_gate"].T) * (h @ w["ffn_up"].T)
    return h + reduce(act @ w["ffn_down"].T), q, k


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = synth.make_activation(1, SPEC.d_model, seed=1, name="tp.x")[0].astype(np.float64)

        def reduce(part):
            t = torch.from_numpy(np.ascontiguousarray(part))
            dist.all_reduce(t)
            return t.numpy()

        y, _, _ = _block(x, {k: v.astype(np.float64) for k, v in _block_parts(rank, world).items()}, reduce)
        # greedy token over a vocabulary sharded by rows: local (value, index) candidates, gathered
        a, b = ll.shard_ranges(SPEC, rank, world)["output"][1:]
        head = oracle.dequant(SPEC.embd_fmt, synth.make_weight(SPEC.embd_fmt, SPEC.vocab, SPEC.d_model, seed=0,
                                                               name="output.weight"), SPEC.vocab, SPEC.d_model)
        logits = head[a:b].astype(np.float64) @ y
        cand = torch.tensor([float(logits.max()), float(a + int(np.argmax(logits)))], dtype=torch.float64)
        gathered = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(gathered, cand)
        best = max(gathered, key=lambda c: (c[0].item(), -c[1].item()))
        if rank == 0:
            q.put((y, int(best[1].item())))
    finally:
        dist.destroy_process_group()


def test_two_rank_block_matches_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    y_tp, tok_tp = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x = synth.make_activation(1, SPEC.d_model, seed=1, name="tp.x")[0].astype(np.float64)
    y, _, _ = _block(x, {k: v.astype(np.float64) for k, v in _block_parts(0, 1).items()}, lambda t: t)
    assert np.allclose(y_tp, y, rtol=1e-10, atol=1e-10)
    head = oracle.dequant(SPEC.embd_fmt, synth.make_weight(SPEC.embd_fmt, SPEC.vocab, SPEC.d_model, seed=0,
                                                           name="output.weight"), SPEC.vocab, SPEC.d_model)
    assert tok_tp == int(np.argmax(head.astype(np.float64) @ y))


def test_shard_plan_rejects_cut_blocks_and_uneven_heads():
    # 7B ffn_down in a K-quant cannot be cut in two: 11008 / 2 = 5504 is not a multiple of 256
    bad = ll.LlamaSpec(1, 4096, 32, 32, 128, 11008, 32000, linear_fmt=synth.Q4_0, down_fmt=synth.Q4_K)
    with pytest.raises(ValueError):
        ll.shard_ranges(bad, 0, 2)
    with pytest.raises(ValueError):
        ll.shard_ranges(ll.SPEC_70B, 0, 16)   # 8 kv heads do not divide over 16 ranks
    r = ll.shard_ranges(ll.SPEC_7B, 7, 8)
    assert r["ffn_down"] == ("cols", 7 * 1376, 8 * 1376) and r["attn_q"] == ("rows", 7 * 512, 8 * 512)

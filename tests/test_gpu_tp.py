"""Tensor-parallel decoder on two GPUs: same greedy tokens as one GPU (skipped with < 2 GPUs).

Each rank is a child process with its own GPU; NCCL's in-switch reduction is switched off
for the test (NCCL_NVLS_ENABLE=0)."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, json
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
from litenn_b200 import capi, synth, llama as ll
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
spec = ll.LlamaSpec(n_layers=3, d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=1024,
                    linear_fmt=synth.Q4_0, embd_fmt=synth.Q6_K, max_seq=64, max_prefill=32)
s = torch.cuda.Stream(); torch.cuda.set_stream(s)
m = ll.LlamaModel(spec, device=rank, tp_rank=rank, tp_size=world, stream=s.cuda_stream, seed=0)
if world > 1:
    path = ll.find_nccl_library()
    box = [ll.nccl_unique_id(path) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    m.tp_init(path, box[0])
    if os.environ.get("QMM_TEST_PEER_EXCHANGE") == "1":
        records = [None] * world
        dist.all_gather_object(records, m.tp_export())
        m.tp_import(records)
prompt = synth.make_token_ids(24, spec.vocab, seed=3, name="tp-prompt")
toks = [m.prefill(prompt)] + m.decode(12).tolist()
m.reset()                                     # a collective on tensor-parallel models
again = [m.prefill(prompt)] + m.decode(12).tolist()
assert again == toks, (again, toks)
assert capi.kernel_status(rank) == 0
if rank == 0:
    print("TOKENS " + json.dumps(toks))
if os.environ.get("QMM_TEST_BATCH", "0") != "0":          # batched decode: sums and candidates travel through NCCL
    B = int(os.environ["QMM_TEST_BATCH"])
    m.reset()
    m.batch_create(B, 8)
    firsts = [m.batch_prefill(b, synth.make_token_ids(6 + 3 * b, spec.vocab, seed=20 + b, name="tp-batch")) for b in range(B)]
    bt = m.batch_decode(8)
    assert capi.kernel_status(rank) == 0
    if rank == 0:
        print("BATCH " + json.dumps([firsts] + bt.tolist()))
m.close()
dist.destroy_process_group()
"""


def run(world, tmp_path, peer_exchange=False, batch=0, prefix="TOKENS "):
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", QMM_TEST_PEER_EXCHANGE="1" if peer_exchange else "0",
               QMM_TEST_BATCH=str(batch))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith(prefix)][-1]
    return line[len(prefix):]


@pytest.mark.parametrize("peer_exchange", [False, True], ids=["nccl-all-reduce", "peer-exchange"])
def test_tp2_tokens_equal_single_gpu(tmp_path, peer_exchange):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    assert run(2, tmp_path, peer_exchange) == run(1, tmp_path)


def test_tp2_batched_decode_equals_single_gpu(tmp_path):
    """Batch of 5 sequences with different prompt lengths: two ranks (NCCL sums of [5, d] rows, all-gather of
    the arg-max candidates) give the tokens of one GPU."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    assert run(2, tmp_path, batch=5, prefix="BATCH ") == run(1, tmp_path, batch=5, prefix="BATCH ")

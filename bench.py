#!/usr/bin/env python
"""Benchmark of the block-quantized matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (config.workload = "llama7b_q4_0_decode_b1"): the random-init 7B-shape
LLaMA decoder of the benchmark configurations (32 layers, d 4096, 32 heads, FFN 11008,
vocab 32000; Q4_0 linears, Q6_K embeddings/output, fp16 KV cache), a 512-token prompt
through the tcgen05 prefill path, then greedy decode at batch 1.  One *step* is one
decoded token; ``value`` is tokens per second over K steps after W warm-up steps, with
N > 1 as tensor parallelism over N GPUs (weights sharded; the two per-block sums after
attention-out and FFN-down travel as packets over peer memory, NCCL only for set-up,
prefill and the arg-max gather), so scaling is "strong".  The 3.75 GB of weights
read per token are far larger than L2.  ``e2e`` drives every token from the host (token
H2D, step, token D2H, synchronize).

The same line carries the first half of the metric, the Q4_0 FFN GEMV W[11008,4096] at
batch 1 ("gemv"), and ``roofline`` for the kernel that dominates both: the batch-1 Q4_0
matvec, timed alone over 12 weight copies (304 MB > 2 x L2) visited round-robin.

``--impl reference`` times the CPU restatement of LiteNN's own path on the host cores
(dequantize once, then the fp32 i-k-j MatMul loop) for one layer's linears plus the
output head on row samples, and extrapolates to the 32 layers.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from litenn_b200 import synth  # noqa: E402

N_OUT, K_IN = 11008, 4096          # W[11008, 4096]: the "4096x11008" FFN projection
BATCH = 1
WEIGHT_BYTES = N_OUT * (K_IN // 32) * 18
ALGO_BYTES = WEIGHT_BYTES + 4 * BATCH * (K_IN + N_OUT)   # 25,422,848 B
COPIES = 12                        # 12 x 25.4 MB = 304 MB > 2 x L2
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one gemv_kernel launch (ncu
# capture summarised under profiles/); None until measured.
NCU_TRAFFIC_BYTES = 25385728


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": float(np.median(sm)) if sm else None,
            "sm_max_mhz": float(max(smax)) if smax else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


DECODE_WEIGHT_BYTES = 32 * 202375168 * 18 // 32 + 131072000 * 210 // 256   # 3,750,273,024 B per token
PROMPT_LEN = 512


def cpu_linear_seconds(n, k, m, threads, rows):
    """Seconds LiteNN's CPU MatMul (Device.h:645-658) needs for x[m,k] @ Wt[k,n], measured on
    `rows` of the n output columns (the i-k-j loop is linear in n) and scaled up."""
    import oracle
    rng = np.random.default_rng(0)
    wt = rng.standard_normal((k, rows)).astype(np.float32)     # an already dequantized, transposed weight
    x = rng.standard_normal((m, k)).astype(np.float32)
    oracle.matmul_ikj(x, wt, threads=threads)
    t0 = time.perf_counter()
    reps = 2
    for _ in range(reps):
        oracle.matmul_ikj(x, wt, threads=threads)
    return (time.perf_counter() - t0) / reps * (n / rows)


def cpu_decode_baseline(threads):
    """tok/s of the reference CPU path for the 7B shape, extrapolated from one layer's seven
    linears plus the output head, each timed on a sample of its output rows."""
    d, ffn, vocab = 4096, 11008, 32000
    t_layer = 4 * cpu_linear_seconds(d, d, 1, threads, 1024)             # q, k, v, o
    t_layer += 2 * cpu_linear_seconds(ffn, d, 1, threads, 1376)          # gate, up
    t_layer += cpu_linear_seconds(d, ffn, 1, threads, 1024)              # down
    t_head = cpu_linear_seconds(vocab, d, 1, threads, 2000)
    t_token = 32 * t_layer + t_head
    t_gemv = cpu_linear_seconds(N_OUT, K_IN, 1, threads, 1376)
    return {
        "value": 1.0 / t_token, "unit": "tok/s", "cores": threads, "kind": "port",
        "sample": ("fp32 i-k-j MatMul loop (Device.h:645-658) on dequantized weights: one layer's seven linears "
                   "(1024-1376 of their output rows each, scaled linearly) x 32 layers + the output head "
                   "(2000 of 32000 rows); one-off dequantization and the interpreter's per-run weight copy excluded; "
                   "extrapolated from one layer"),
        "seconds_per_token": t_token,
        "gemv_gbs": ALGO_BYTES / t_gemv / 1e9,
    }


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    import oracle
    threads = oracle.max_threads()
    t0 = time.perf_counter()
    res = cpu_decode_baseline(threads)
    line = {
        "impl": "reference",
        "metric": "7B-shape Q4_0 batch-1 decode tok/s",
        "value": res["value"],
        "unit": "tok/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": res["seconds_per_token"] * 1e3,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "llama7b_q4_0_decode_b1", "prompt": PROMPT_LEN, "batch": 1,
                   "l2": "CPU run; a step is one token extrapolated from one layer's linears"},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "gemv": {"value": res["gemv_gbs"], "unit": "GB/s", "workload": "q4_0_gemv_4096x11008_b1"},
        "e2e": {"value": res["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))
    return 0


def gemv_micro(torch, capi, local, side, stream, steps, warmup):
    """The Q4_0 FFN GEMV at batch 1 over 12 weight copies: (public call, kernel alone) in us."""
    weights = []
    for i in range(COPIES):
        payload = synth.make_weight(synth.Q4_0, N_OUT, K_IN, seed=0, name=f"bench.w{i % 2}")
        weights.append(capi.Weight.from_host(synth.Q4_0, payload, N_OUT, K_IN, device=local, stream=stream))
    x = torch.from_numpy(synth.make_activation(BATCH, K_IN, seed=0, name="bench.x")).cuda()
    ys = [torch.empty((BATCH, N_OUT), dtype=torch.float32, device="cuda") for _ in range(COPIES)]
    packed = torch.empty(capi.packed_activation_bytes(K_IN, BATCH), dtype=torch.uint8, device="cuda")
    capi.pack_activations(x.data_ptr(), BATCH, K_IN, packed.data_ptr(), device=local, stream=stream)

    def step_full():
        for w, y in zip(weights, ys):
            w.gemv_f32(x.data_ptr(), y.data_ptr(), BATCH, stream)

    def step_kernel():
        for w, y in zip(weights, ys):
            w.gemv_packed(packed.data_ptr(), y.data_ptr(), BATCH, stream)

    out = []
    for fn in (step_full, step_kernel):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            fn()
        for _ in range(max(3, warmup)):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) * 1e3 / (steps * COPIES))
    capi.kernel_status(local)
    y = ys[-1].cpu().numpy()
    if not np.isfinite(y).all() or not np.abs(y).max() > 0:
        raise SystemExit("bench.py: GEMV produced non-finite or all-zero output")
    for w in weights:
        w.destroy()
    return out[0], out[1]


def gemm_micro(torch, capi, local, stream, steps, warmup):
    """Prefill GEMM of configs[2]: M=512 bf16 tokens x K=4096 x N=14336 in Q4_K and Q6_K.
    Four weight copies per format are visited round-robin (4 x 33-48 MB > L2)."""
    m, k, n = 512, 4096, 14336
    out = {}
    x = torch.from_numpy(synth.make_activation(m, k, seed=0, name="bench.gemm.x")).cuda().to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    for fmt, name in ((synth.Q4_K, "q4_k"), (synth.Q6_K, "q6_k")):
        payload = synth.make_weight(fmt, n, k, seed=0, name="bench.gemm.w")
        ws = [capi.Weight.from_host(fmt, payload, n, k, device=local, stream=stream) for _ in range(4)]
        for i in range(max(3, warmup)):
            ws[i % 4].gemm_bf16(x.data_ptr(), y.data_ptr(), m, capi.OUT_F32, stream)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            ws[i % 4].gemm_bf16(x.data_ptr(), y.data_ptr(), m, capi.OUT_F32, stream)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / steps
        out[name] = {"us": us, "tflops": 2.0 * m * n * k / (us * 1e-6) / 1e12}
        for w in ws:
            w.destroy()
    capi.kernel_status(local)
    if not torch.isfinite(y).all():
        raise SystemExit("bench.py: GEMM produced non-finite output")
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from litenn_b200 import capi
    from litenn_b200 import llama as ll

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    capi.load()
    side = torch.cuda.Stream()
    torch.cuda.set_stream(side)
    stream = side.cuda_stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.device_only == "gemm":
        res = gemm_micro(torch, capi, local, stream, max(4, args.steps), args.warmup)
        if rank == 0:
            print(json.dumps({"device_only": "gemm", "workload": "prefill_gemm_m512_k4096_n14336", **res}))
        return 0
    gemv_steps = 50
    full_us, kernel_us = (0.0, 0.0) if args.device_only in ("decode", "decode70b") else gemv_micro(torch, capi, local, side, stream,
                                                                                    gemv_steps, 3)
    if args.device_only == "gemv":
        if rank == 0:
            print(json.dumps({"device_only": "gemv", "us_per_gemv": full_us, "us_per_gemv_kernel": kernel_us}))
        return 0

    # ---- the decoder -----------------------------------------------------------------
    K, W = args.steps, max(3, args.warmup)
    e2e_steps = min(K, 32)
    import dataclasses
    spec, prompt_len = ll.SPEC_7B, PROMPT_LEN
    if args.device_only == "decode70b":   # configs[4]: 70B shape, GQA, Q4_K / Q6_K, 1024-token prompt
        spec, prompt_len = ll.SPEC_70B, 1024
        if args.layers:
            spec = dataclasses.replace(spec, n_layers=args.layers)
    spec = dataclasses.replace(spec, max_seq=prompt_len + W + K + e2e_steps + 16, max_prefill=prompt_len)
    model = ll.LlamaModel(spec, device=local, tp_rank=rank, tp_size=world, stream=stream, share_layer_payloads=True)
    if world > 1:
        path = ll.find_nccl_library()
        box = [ll.nccl_unique_id(path) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        model.tp_init(path, box[0])
        records = [None] * world
        dist.all_gather_object(records, model.tp_export())
        model.tp_import(records)                  # decode sums the per-block partials over peer memory
    prompt = synth.make_token_ids(prompt_len, spec.vocab, seed=0, name="prompt")
    torch.cuda.synchronize()
    t_prefill = time.perf_counter()
    first = model.prefill(prompt)        # returns after the first token has come back to the host
    prefill_ms = (time.perf_counter() - t_prefill) * 1e3
    model.decode(W)                      # warm-up steps (the first one also builds the CUDA graph)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    model.decode_enqueue(K)
    stop.record()
    barrier()
    ms_total = start.elapsed_time(stop)
    if args.device_only in ("decode", "decode70b"):  # the timed region alone (ncu launch lists, 70B runs)
        t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            sampler.stop()
            print(json.dumps({"device_only": args.device_only, "tok_s": K / (float(t.cpu()[0]) * 1e-3), "steps": K,
                              "warmup": W, "n_gpus": world, "layers": spec.n_layers, "d_model": spec.d_model}))
        model.close()
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- end to end: every token crosses the host ---------------------------------------
    tok = first
    for _ in range(2):
        tok = model.step_host(tok)
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(e2e_steps):
        tok = model.step_host(tok)
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop)
    clocks = sampler.stop() if rank == 0 else None
    capi.kernel_status(local)
    if not (0 <= tok < spec.vocab):
        raise SystemExit("bench.py: decoder produced an out-of-range token")

    times = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = (float(v) for v in times.cpu())

    if rank == 0:
        peak, peak_kind = measured_peak()
        value = K / (ms_total * 1e-3)
        achieved = ALGO_BYTES / (kernel_us * 1e-6) / 1e9
        # per block: norm+pack, qkv matvec, fused attention, attn_output matvec, norm+pack, gate|up
        # matvec, SwiGLU+pack, down matvec; per token also: embedding row, final norm, output
        # matvec, arg-max, commit (the NCCL gather of arg-max candidates at N > 1 is not ours)
        kernels_per_token = 1 + spec.n_layers * 8 + 4
        line = {
            "metric": "7B-shape Q4_0 batch-1 decode tok/s",
            "value": value,
            "unit": "tok/s",
            "n_gpus": world,
            "steps": K,
            "warmup": W,
            "ms_per_step": ms_total / K,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "int8 tensor-core products, fp32 accumulate (decode); bf16 tcgen05 (prefill)",
            "data": "synthetic",
            "config": {"workload": "llama7b_q4_0_decode_b1", "layers": 32, "d_model": 4096, "heads": 32, "ffn": 11008,
                       "vocab": 32000, "prompt": PROMPT_LEN, "batch": 1, "kv_cache": "fp16",
                       "parallelism": f"tp{world}" if world > 1 else "single",
                       "launch": "one CUDA graph per token",
                       "l2": "inputs larger than L2: 3.75 GB of weights are read per token",
                       "prefill_ms_first_call": prefill_ms,
                       "weight_bytes_per_token": DECODE_WEIGHT_BYTES,
                       "frac_of_weight_stream_bound": value / (peak * 1e9 / DECODE_WEIGHT_BYTES * world),
                       "bound_tok_s_at_peak": peak * 1e9 / DECODE_WEIGHT_BYTES * world},
            "gemv": {"metric": "Q4_0 GEMV achieved HBM GB/s", "workload": "q4_0_gemv_4096x11008_b1",
                     "value": ALGO_BYTES / (full_us * 1e-6) / 1e9, "unit": "GB/s", "us_per_call": full_us,
                     "copies": COPIES, "algorithmic_bytes": ALGO_BYTES,
                     "note": "public call qmm_gemv_f32 = pack_x + gemv, one CUDA graph of 12 calls"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES, "peak_source": f"of {peak_kind}",
                         "frac_of_nominal_8tbs": achieved / 8000.0,
                         "kernel": "gemv_kernel<Q4_0, batch 1> on W[11008,4096]", "us_per_launch": kernel_us,
                         "how": "CUDA events around graph replays of 12 back-to-back launches of this kernel alone "
                                "(12 weight copies = 304 MB > 2 x L2), activations packed once"},
            "e2e": {"value": e2e_steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 4,
                    "d2h_bytes_per_step": 4, "steps": e2e_steps},
            "gpu_launches": kernels_per_token * (K + e2e_steps) * world,
            "clocks": clocks,
        }
        if world == 1:
            cpu = cpu_decode_baseline(1)
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    model.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--device-only", choices=["gemv", "decode", "gemm", "decode70b"], default=None,
                    help="run one device-timed part alone (used for ncu captures): the Q4_0 GEMV, the decode\n"
                         "steps, or the prefill GEMM of configs[2]")
    ap.add_argument("--layers", type=int, default=0, help="with --device-only decode70b: blocks to build (default 80)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())

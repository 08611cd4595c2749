#!/usr/bin/env python
"""Benchmark of the block-quantized matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload = "q4_0_gemv_4096x11008_b1"): the FFN-shaped Q4_0
GEMV of the benchmark configurations — weight W[11008,4096] in Q4_0 (the
"4096x11008" linear), fp32 activation vector, batch 1.  One *step* is one pass
over ``copies`` distinct copies of the weight (280 MB in total, more than twice
the 126 MB L2, so every launch streams its weights from HBM), i.e. ``copies``
GEMV calls.  ``value`` is algorithmic bytes moved per second with inputs already
resident in HBM; ``e2e`` is the same metric through the host-buffer entry point
(activation H2D and result D2H inside the timed region, one synchronizing call
per GEMV).  With N > 1 every rank runs the same workload on its own GPU (the
single-matrix GEMV shards into independent replicas; no collective on the data
path) and the values add up.

``--impl reference`` times the CPU restatement of LiteNN's own path on the host
cores: dequantize once, then the fp32 i-k-j MatMul loop.
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
NCU_TRAFFIC_BYTES = 25385000


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


def cpu_reference_run(steps: int, warmup: int, threads: int, sample_rows: int):
    """LiteNN's CPU path on a bounded sample: `sample_rows` output rows of the
    11008x4096 weight (the i-k-j loop's cost is linear in N), fp32, `threads` threads."""
    import oracle
    payload = synth.make_weight(synth.Q4_0, sample_rows, K_IN, seed=0, name="bench.w0")
    x = synth.make_activation(BATCH, K_IN, seed=0, name="bench.x")
    t0 = time.perf_counter()
    w = oracle.dequant(synth.Q4_0, payload, sample_rows, K_IN)      # one-off, reported separately
    wt = oracle.transpose(w)
    dequant_s = time.perf_counter() - t0
    for _ in range(warmup):
        oracle.matmul_ikj(x, wt, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.matmul_ikj(x, wt, threads=threads)
    per_call = (time.perf_counter() - t0) / steps
    full_call_s = per_call * (N_OUT / sample_rows)
    return {
        "value": ALGO_BYTES / full_call_s / 1e9,
        "unit": "GB/s",
        "cores": threads,
        "kind": "port",
        "sample": (f"{sample_rows} of {N_OUT} output rows of the Q4_0 {N_OUT}x{K_IN} weight, batch {BATCH}; "
                   f"fp32 i-k-j loop (Device.h:645-658) after a one-off dequant+transpose "
                   f"({dequant_s * 1e3:.1f} ms for the sample, excluded); scaled linearly to the full matrix"),
        "ms_per_call_full": full_call_s * 1e3,
    }


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    import oracle
    threads = oracle.max_threads()
    rows = 2752  # a quarter of the matrix
    t0 = time.perf_counter()
    res = cpu_reference_run(max(1, args.steps), max(1, args.warmup), threads, rows)
    line = {
        "impl": "reference",
        "metric": "Q4_0 GEMV achieved HBM GB/s",
        "value": res["value"],
        "unit": "GB/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": res["ms_per_call_full"] * COPIES,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "q4_0_gemv_4096x11008_b1", "n": N_OUT, "k": K_IN, "batch": BATCH,
                   "l2": "CPU run; a step is `copies` matvecs scaled from a row sample", "copies": COPIES},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))
    return 0


def run_ours(args):
    import torch
    import torch.distributed as dist
    from litenn_b200 import capi

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    capi.load()

    # All work runs on one side stream so that a step can be captured into a CUDA graph
    # (decode replays graphs; per-call launch cost from Python would hide the kernels).
    side = torch.cuda.Stream()
    torch.cuda.set_stream(side)
    stream = side.cuda_stream
    weights = []
    for i in range(COPIES):
        payload = synth.make_weight(synth.Q4_0, N_OUT, K_IN, seed=0, name=f"bench.w{i}")
        weights.append(capi.Weight.from_host(synth.Q4_0, payload, N_OUT, K_IN, device=local, stream=stream))
    x_host = synth.make_activation(BATCH, K_IN, seed=0, name="bench.x")
    x = torch.from_numpy(x_host).cuda()
    ys = [torch.empty((BATCH, N_OUT), dtype=torch.float32, device="cuda") for _ in range(COPIES)]

    def step():
        for w, y in zip(weights, ys):
            w.gemv_f32(x.data_ptr(), y.data_ptr(), BATCH, stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------------
    step()                      # allocates the per-stream scratch before capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    run_step = graph.replay
    for _ in range(max(3, args.warmup)):
        run_step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # enough repetitions of the K-step region for the clock sampler to see load
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        run_step()
    stop.record()
    barrier()
    ms_total = start.elapsed_time(stop)

    # ---- the dominant kernel alone: matvecs on activations packed once ---------------
    packed = torch.empty(capi.packed_activation_bytes(K_IN, BATCH), dtype=torch.uint8, device="cuda")
    capi.pack_activations(x.data_ptr(), BATCH, K_IN, packed.data_ptr(), device=local, stream=stream)

    def step_kernel():
        for w, y in zip(weights, ys):
            w.gemv_packed(packed.data_ptr(), y.data_ptr(), BATCH, stream)

    step_kernel()
    torch.cuda.synchronize()
    kgraph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(kgraph, stream=side):
        step_kernel()
    for _ in range(max(3, args.warmup)):
        kgraph.replay()
    barrier()
    k_start, k_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k_start.record()
    for _ in range(args.steps):
        kgraph.replay()
    k_stop.record()
    barrier()
    kernel_ms_total = k_start.elapsed_time(k_stop)
    capi.kernel_status(local)

    if args.device_only:
        if rank == 0:
            sampler.stop()
            print(json.dumps({"device_only": True, "us_per_gemv": ms_total * 1e3 / (args.steps * COPIES),
                              "us_per_gemv_kernel": kernel_ms_total * 1e3 / (args.steps * COPIES)}))
        return 0

    # ---- end-to-end through the host-buffer entry point --------------------------------
    x_pin = torch.from_numpy(x_host.copy()).pin_memory()
    y_pin = torch.empty((BATCH, N_OUT), dtype=torch.float32).pin_memory()
    x_np, y_np = x_pin.numpy(), y_pin.numpy()

    def step_e2e():
        for w in weights:
            w.gemv_f32_host(x_np, y_np, BATCH, stream)

    for _ in range(3):
        step_e2e()
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        step_e2e()
    e_stop.record()
    barrier()
    e2e_ms_total = e_start.elapsed_time(e_stop)
    clocks = sampler.stop() if rank == 0 else None

    # correctness guard on the last result (cheap, outside the timed regions)
    y_last = ys[-1].cpu().numpy()
    if not np.isfinite(y_last).all() or not np.abs(y_last).max() > 0:
        raise SystemExit("bench.py: GEMV produced non-finite or all-zero output")
    if not np.allclose(y_np, y_last, rtol=1e-5, atol=1e-6):
        raise SystemExit("bench.py: host-buffer path disagrees with the device path")

    times = torch.tensor([ms_total, e2e_ms_total, kernel_ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms_total, kernel_ms_total = (float(v) for v in times.cpu())

    if rank == 0:
        launches_per_rank = args.steps * COPIES
        gemv_per_s = world * launches_per_rank / (ms_total * 1e-3)
        value = gemv_per_s * ALGO_BYTES / 1e9
        e2e_value = world * launches_per_rank / (e2e_ms_total * 1e-3) * ALGO_BYTES / 1e9
        peak, peak_kind = measured_peak()
        per_launch_us = ms_total * 1e3 / launches_per_rank
        kernel_us = kernel_ms_total * 1e3 / launches_per_rank
        achieved = ALGO_BYTES / (kernel_us * 1e-6) / 1e9
        cpu = cpu_reference_run(steps=3, warmup=1, threads=1, sample_rows=1376) if world == 1 else None
        line = {
            "metric": "Q4_0 GEMV achieved HBM GB/s",
            "value": value,
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(3, args.warmup),
            "ms_per_step": ms_total / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "int8 tensor-core products, fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": "q4_0_gemv_4096x11008_b1", "n": N_OUT, "k": K_IN, "batch": BATCH, "copies": COPIES,
                       "launch": "one CUDA graph per step",
                       "l2": f"inputs larger than L2: {COPIES} weight copies = {COPIES * WEIGHT_BYTES / 1e6:.0f} MB "
                             "visited round-robin",
                       "algorithmic_bytes_per_gemv": ALGO_BYTES, "us_per_gemv": per_launch_us,
                       "parallelism": "replicas" if world > 1 else "single"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES, "peak_source": f"of {peak_kind}",
                         "kernel": "gemv_kernel<Q4_0, batch 1>", "us_per_launch": kernel_us,
                         "how": "CUDA events around K graph replays of `copies` back-to-back launches of this "
                                "kernel alone, on activations packed once"},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": COPIES * BATCH * K_IN * 4,
                    "d2h_bytes_per_step": COPIES * BATCH * N_OUT * 4, "us_per_gemv": e2e_ms_total * 1e3 / launches_per_rank},
            # value region: pack_x + gemv per call; kernel region: gemv; e2e region: pack_x + gemv
            "gpu_launches": (2 + 1 + 2) * launches_per_rank * world,
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--device-only", action="store_true",
                    help="run only the device-resident timed region (used for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())

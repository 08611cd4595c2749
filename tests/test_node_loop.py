"""The block-quantized MatMul pattern executed by stand-ins for LiteNN's two runtimes
(litenn_b200/host/QuantizedGraphRuntime.hpp): a node loop in the order of
Interpreter::RunSubgraphUnchecked (src/LiteNN/Runtime/Interpreter.h:79-114, 325-354) and a payload-record
dispatcher shaped like RunCUDANativeLibraryCall (src/LiteNN/Compiler/CompiledModule.cpp:4114-4180)."""
import os
import subprocess

import numpy as np
import pytest

import oracle
from litenn_b200 import capi, synth
from helpers import REL_TOL

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "native", "node_loop_test.cpp")
EXE = os.path.join(HERE, "native", "node_loop_test")


@pytest.fixture(scope="module")
def node_loop_exe(qmm_lib):
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    deps = [SRC, os.path.join(ROOT, "litenn_b200", "host", "QuantizedGraphRuntime.hpp"),
            os.path.join(ROOT, "litenn_b200", "host", "LiteNNQuantMatMul.hpp"), os.path.join(ROOT, "include", "litenn_qmm.h")]
    if not os.path.exists(EXE) or any(os.path.getmtime(d) > os.path.getmtime(EXE) for d in deps):
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(cuda, "include"), "-o", EXE, SRC,
                        "-L", os.path.join(ROOT, "litenn_b200"), "-lqmm_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
                        "-Wl,-rpath," + os.path.join(ROOT, "litenn_b200"), "-Wl,-rpath," + os.path.join(cuda, "lib64")],
                       check=True)
    return EXE


def test_record_validation_and_node_errors_need_no_gpu(node_loop_exe):
    """Unknown kernel name, missing or unknown feature bit, constant range beyond the payload, wrong argument count,
    and a node whose input was never produced (message carries the node id and kind)."""
    if capi.device_count() > 0:
        pytest.skip("covered by the GPU test")
    r = subprocess.run([node_loop_exe], capture_output=True, text=True)
    assert r.returncode == 77, r.stdout + r.stderr
    assert "SKIP" in r.stdout and "FAIL" not in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K])
@pytest.mark.parametrize("m", [1, 5, 64])
def test_pattern_runs_through_both_runtimes(node_loop_exe, tmp_path, fmt, m):
    n, k = 96, 512
    payload = synth.make_weight(fmt, n, k, seed=7, name="node-loop")
    x = synth.make_activation(m, k, seed=7, name="node-loop-x")
    w = oracle.dequant(fmt, payload, n, k)
    if m <= 16:
        ref = oracle.quantized_matmul(fmt, payload, n, k, x)
    else:   # more than 16 fp32 rows take the tensor-core GEMM: product of the bf16-rounded operands
        ref = oracle.matmul_nk_f64(oracle.fp32_to_bf16_round(x), oracle.fp32_to_bf16_round(w)).astype(np.float32)
    files = {}
    for name, arr in (("payload", payload), ("x", x), ("y", ref), ("w", w)):
        files[name] = str(tmp_path / f"{name}.bin")
        np.ascontiguousarray(arr).tofile(files[name])
    r = subprocess.run([node_loop_exe, str(fmt), str(n), str(k), str(m), files["payload"], files["x"], files["y"], files["w"]],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    out = dict((" ".join(l.split()[:-1]), l.split()[-1]) for l in r.stdout.splitlines())
    assert float(out["node_loop max_rel_err"]) <= REL_TOL
    assert float(out["library_call max_rel_err"]) <= REL_TOL
    assert out["dequant bit_exact"] == "1"

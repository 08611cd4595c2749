"""The LiteNN-facing C++ adapter (litenn_b200/host/LiteNNQuantMatMul.hpp)."""
import os
import subprocess

import numpy as np
import pytest

import oracle
from litenn_b200 import capi, synth
from helpers import REL_TOL

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "native", "adapter_test.cpp")
EXE = os.path.join(HERE, "native", "adapter_test")


@pytest.fixture(scope="module")
def adapter_exe(qmm_lib):
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    deps = [SRC, os.path.join(ROOT, "litenn_b200", "host", "LiteNNQuantMatMul.hpp"),
            os.path.join(ROOT, "include", "litenn_qmm.h")]
    if not os.path.exists(EXE) or any(os.path.getmtime(d) > os.path.getmtime(EXE) for d in deps):
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(cuda, "include"), "-o", EXE, SRC,
                        "-L", os.path.join(ROOT, "litenn_b200"), "-lqmm_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
                        "-Wl,-rpath," + os.path.join(ROOT, "litenn_b200"), "-Wl,-rpath," + os.path.join(cuda, "lib64")],
                       check=True)
    return EXE


def test_adapter_compiles_and_reports_errors_as_exceptions(adapter_exe):
    """Without a GPU the program still checks that a bad row width throws
    std::runtime_error with LiteNN's message, then reports SKIP (exit 77)."""
    if capi.device_count() > 0:
        pytest.skip("covered by the GPU test")
    r = subprocess.run([adapter_exe], capture_output=True, text=True)
    assert r.returncode == 77, r.stdout + r.stderr
    assert "SKIP" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [synth.Q4_0, synth.Q6_K])
@pytest.mark.parametrize("m", [3, 17, 512])
def test_adapter_matmul_matches_oracle(adapter_exe, tmp_path, fmt, m):
    """fp32 activations through the DoBinaryOp-shaped entry: up to 16 rows take the matvec (compared with the
    reference's fp32 product), more rows take the prefill GEMM (compared with the product of the bf16-rounded
    operands, which is what that path computes)."""
    n, k = 160, 1024
    payload = synth.make_weight(fmt, n, k, seed=4, name="adapter")
    x = synth.make_activation(m, k, seed=4, name="adapter-x")
    if m <= 16:
        ref = oracle.quantized_matmul(fmt, payload, n, k, x)
    else:
        ref = oracle.matmul_nk_f64(oracle.fp32_to_bf16_round(x),
                                   oracle.fp32_to_bf16_round(oracle.dequant(fmt, payload, n, k))).astype(np.float32)
    files = {}
    for name, arr in (("payload", payload), ("x", x), ("expected", ref)):
        files[name] = str(tmp_path / f"{name}.bin")
        np.ascontiguousarray(arr).tofile(files[name])
    r = subprocess.run([adapter_exe, str(fmt), str(n), str(k), str(m), files["payload"], files["x"], files["expected"]],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    err = float(r.stdout.split("max_rel_err")[1].split()[0])
    assert err <= REL_TOL

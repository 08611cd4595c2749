"""Failure detection around the prefill collectives, exercised with a stand-in NCCL library
(tests/native/nccl_stub.c) that the C ABI loads by path.  Nothing here faults or hangs a GPU: the
stand-in keeps a stream busy with a sleeping HOST function and reports an asynchronous error, or simply
takes longer than the collective time limit; the library must poll ncclCommGetAsyncError, abort the
communicator, return QMM_E_CUDA and refuse further tensor-parallel work.  Each case runs in its own
process because the NCCL entry points are resolved once per process."""
import os
import subprocess
import sys
import textwrap

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "native", "nccl_stub.c")
LIB = os.path.join(HERE, "native", "libnccl_stub.so")


@pytest.fixture(scope="module")
def stub_lib():
    if not os.path.exists(LIB) or os.path.getmtime(SRC) > os.path.getmtime(LIB):
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-Wall", "-I", os.path.join(cuda, "include"), SRC, "-o", LIB,
                        "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(cuda, "lib64")], check=True)
    return LIB


def run_child(code, env_extra):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), **env_extra)
    return subprocess.run([sys.executable, "-c", textwrap.dedent(code)], capture_output=True, text=True, env=env, cwd=ROOT,
                          timeout=600)


def test_library_is_resolved_by_path_and_missing_symbols_are_refused(stub_lib, tmp_path):
    """No GPU needed: the unique id comes from the stand-in; a library without the entry points is an error."""
    r = run_child(f"""
        from litenn_b200 import llama
        uid = llama.nccl_unique_id({stub_lib!r})
        assert uid.startswith(b"nccl-stub-unique-id"), uid
        print("ok")
    """, {"NCCL_STUB_LOG": str(tmp_path / "log")})
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
    assert (tmp_path / "log").read_text().split() == ["ncclGetUniqueId"]
    empty = tmp_path / "libempty.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-x", "c", "/dev/null", "-o", str(empty)], check=True)
    r = run_child(f"""
        from litenn_b200 import llama, capi
        try:
            llama.nccl_unique_id({str(empty)!r})
        except capi.QmmError as e:
            assert e.code == capi.E_UNSUPPORTED and "lacks a required symbol" in str(e), e
            print("ok")
    """, {})
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


CHILD = """
    import time
    import numpy as np
    from litenn_b200 import llama, capi
    from litenn_b200 import synth
    spec = llama.LlamaSpec(n_layers=1, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=512,
                           linear_fmt=synth.Q4_0, embd_fmt=synth.Q6_K, max_seq=64, max_prefill=32)
    model = llama.LlamaModel(spec, seed=0, tp_rank=0, tp_size=2)
    model.tp_init({lib!r}, llama.nccl_unique_id({lib!r}))
    model.set_collective_timeout({timeout_ms})
    prompt = np.arange(8, dtype=np.int32) % spec.vocab
    t0 = time.perf_counter()
    try:
        model.prefill(prompt)
        print("no error")
    except capi.QmmError as e:
        print("code", e.code, "|", e)
    print("elapsed", time.perf_counter() - t0)
    try:
        model.prefill(prompt)
        print("second prefill ran")
    except capi.QmmError as e:
        print("second", e.code, "|", e)
    model.close()
    print("status", capi.kernel_status(0))
"""


@pytest.mark.gpu
def test_async_error_aborts_the_communicator(stub_lib, tmp_path):
    log = tmp_path / "log"
    r = run_child(CHILD.format(lib=stub_lib, timeout_ms=20000),
                  {"NCCL_STUB_BUSY_MS": "300", "NCCL_STUB_ASYNC_ERROR": "6", "NCCL_STUB_LOG": str(log)})
    assert r.returncode == 0, r.stdout + r.stderr
    assert "code -2 |" in r.stdout, r.stdout                                     # QMM_E_CUDA
    assert "NCCL reported an asynchronous error (6); communicator aborted" in r.stdout
    assert "second" in r.stdout and "before qmm_llama_tp_init" in r.stdout     # refuses further tensor-parallel work
    assert "status 0" in r.stdout                                               # no kernel gave up; the GPU is healthy
    calls = log.read_text().split()
    assert "ncclCommAbort" in calls and "ncclCommDestroy" not in calls


@pytest.mark.gpu
def test_collective_slower_than_the_limit_is_given_up(stub_lib, tmp_path):
    log = tmp_path / "log"
    r = run_child(CHILD.format(lib=stub_lib, timeout_ms=50), {"NCCL_STUB_BUSY_MS": "400", "NCCL_STUB_LOG": str(log)})
    assert r.returncode == 0, r.stdout + r.stderr
    assert "did not finish within 50 ms; communicator aborted" in r.stdout
    elapsed = float(r.stdout.split("elapsed")[1].split()[0])
    assert elapsed < 5.0
    assert "ncclCommAbort" in log.read_text().split()


@pytest.mark.gpu
def test_healthy_stand_in_lets_prefill_finish(stub_lib, tmp_path):
    r = run_child(CHILD.format(lib=stub_lib, timeout_ms=20000), {"NCCL_STUB_BUSY_MS": "5", "NCCL_STUB_LOG": str(tmp_path / "log")})
    assert r.returncode == 0, r.stdout + r.stderr
    assert "no error" in r.stdout and "second prefill ran" in r.stdout
    assert "ncclCommAbort" not in (tmp_path / "log").read_text().split()

"""Builds ``libqmm_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Each ``csrc/*.cu`` is compiled to an object file (in parallel, only when stale)
and linked into ``litenn_b200/libqmm_b200.so``.  ``-Xptxas -v`` output is kept in
``litenn_b200/build/ptxas.log``.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libqmm_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "-I", INCLUDE,
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libqmm_b200.so")


def _host_compiler_flags() -> list[str]:
    # nvcc must drive the distribution's g++ (the image also carries a wrapper compiler).
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def _deps_mtime() -> float:
    newest = 0.0
    for root in (CSRC, INCLUDE):
        for f in os.listdir(root):
            if f.endswith((".h", ".cuh")):
                newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    return newest


def _compile(src: str, obj: str) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, *_host_compiler_flags(), "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return f"==== {os.path.basename(src)}\n{r.stderr}"


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_m = _deps_mtime()
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(BUILD, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_m):
            jobs.append((s, o))
    logs = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(lambda so: _compile(*so), jobs):
                logs.append(log)
        with open(os.path.join(BUILD, "ptxas.log"), "a") as f:
            f.write("\n".join(logs) + "\n")
        if verbose:
            print("\n".join(logs))
    if jobs or not os.path.exists(LIB):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", *_host_compiler_flags(),
               "-shared", "-o", LIB, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))

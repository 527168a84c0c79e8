"""Builds libllm_b200.so in-tree with nvcc for sm_100a (no torch extension machinery).

Usage: python llm.cu_b200/build.py [--force]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libllm_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
SOURCES = [
    "csrc/runtime.cu",
    "csrc/misc.cu",
    "csrc/gemv.cu",
    "csrc/attn_decode.cu",
    "csrc/decode_step.cu",
    "csrc/gemm_tc.cu",
    "csrc/gemm_smallm.cu",
    "csrc/prefill.cu",
    "csrc/sampler.cu",
    "csrc/tp_rows.cu",
    "host/model.cu",
    "host/engine.cu",
    "host/safetensor.cpp",
    "host/sampler.cpp",
]
HEADERS = [
    "csrc/common.cuh",
    "csrc/gemv_common.cuh",
    "csrc/gemm_common.cuh",
    "csrc/tp_common.cuh",
    "csrc/mma_common.cuh",
    "host/host_internal.h",
    "../include/llm_b200.h",
    "../include/llama3.h",
    "../include/llm_b200_synth.h",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--threads", "2",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compiles every source for sm_100a and links the shared library. Returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(HERE, h) for h in HEADERS] + [os.path.abspath(__file__)]
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in SOURCES:
        path = os.path.join(HERE, src)
        obj = os.path.join(OBJ_DIR, src.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-x", "cu"] if src.endswith(".cpp") else []) + ["-c", path, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n%s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
        return r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(4, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or force or _stale(LIB, objs):
        run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))

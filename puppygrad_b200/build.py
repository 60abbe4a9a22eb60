"""Builds `libpuppygrad_b200.so` in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m puppygrad_b200.build [--force]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libpuppygrad_b200.so")
OBJ_DIR = os.path.join(CSRC, "build")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-I", INCLUDE, "-I", CSRC]
# developer aid: extra compiler flags (e.g. PG_NVCC_EXTRA="-DPG_DEV_TRACE"); rebuild with --force after changing it
NVCC_FLAGS += os.environ.get("PG_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build puppygrad_b200")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return hs + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    newest_header = max(os.path.getmtime(h) for h in _headers())
    objs, rebuilt = [], False
    for src in _sources():
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(path), newest_header)
        if not stale:
            continue
        if src.endswith(".cu"):
            cmd = [nvcc, *NVCC_FLAGS, "-c", path, "-o", obj]
        else:
            cmd = [os.environ.get("CXX", "g++"), *CXX_FLAGS, "-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
        rebuilt = True
    if rebuilt or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs,
               "-cudart", "static", "-lpthread"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))

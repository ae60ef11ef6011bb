"""Compile the CUDA kernels and their C ABI into ``trigrad_b200/libtrigrad_b200.so`` (sm_100a only).

The library is built in-tree with plain nvcc (no torch headers: the ABI is C).  cudart is linked
statically so that the shared object is self-contained.

Usage: python -m trigrad_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtrigrad_b200.so")
SOURCES = ["tg_binning.cu", "tg_sort.cu", "tg_tilesort.cu", "tg_blend.cu", "tg_project.cu", "tg_clip.cu", "tg_api.cu"]
HEADERS = [os.path.join(CSRC, "tg_common.cuh"), os.path.join(CSRC, "tg_radix.cuh"), os.path.join(HERE, "..", "include", "trigrad_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    flags += os.environ.get("TG_EXTRA_NVCC_FLAGS", "").split()   # extra compiler flags for experiments

    def one(src: str) -> str:
        obj = os.path.join(objdir, src + ".o")
        cmd = [_nvcc(), "-c"] + flags + [os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(one, SOURCES))
    tmp = LIB + ".tmp"     # link beside the target and rename: a reader never sees a half-written library
    cmd = [_nvcc(), "-shared", "-o", tmp] + objs + ["-cudart", "static"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))

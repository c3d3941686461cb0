"""Builds libpolaris_s14_cuda.so (sm_100a only) next to this file with nvcc.

Run as ``python -m colormlm_b200.build``.  The library is built in-tree so that it
travels with the source tree; there is no JIT cache and no other architecture.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libpolaris_s14_cuda.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)
SOURCES = ["s14_kernels.cu", "s14_moe_umma.cu", "s14_moe_block.cu", "s14_glue.cu", "s14_api.cu", "s14_host.cpp"]
HEADERS = ["s14_internal.h", "s14_device.cuh", "s14_umma.cuh", "s14_host.hpp", os.path.join("..", "..", "include", "polaris_s14_cuda.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-ccbin", shutil.which("g++") or "g++",
        "-o", LIB_PATH,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

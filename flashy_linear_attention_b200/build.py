"""Builds libflashlinear_sm100.so in-tree with nvcc for sm_100a.

Usage: python -m flashy_linear_attention_b200.build [--force]
The library has no Python or torch dependency; it links the static CUDA runtime only.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libflashlinear_sm100.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)

SOURCES = ["fla_api.cu"]
HEADERS = ["fla_kernel.cuh", "fla_wide_kernel.cuh", "fla_normalize.cuh", "fla_taylor.cuh", "ptx.cuh", os.path.join("..", "..", "include", "flashlinear_sm100.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build " + LIB_NAME)
    return nvcc


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    for f in SOURCES + HEADERS:
        if os.path.getmtime(os.path.join(CSRC, f)) > built:
            return True
    return False


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the CUDA sources if the library is missing or older than a source file."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [find_nvcc()] + NVCC_FLAGS
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

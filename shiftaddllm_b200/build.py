"""Builds ``libsal_lutgemm.so`` (CUDA kernels + C ABI) for sm_100a, in-tree.

Usage: ``python -m shiftaddllm_b200.build [--force] [--verbose]``.
nvcc cross-compiles without a GPU.  The library has no dependency on torch.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
SRCS = [os.path.join(PKG_DIR, "csrc", name) for name in ("sal_lutgemm.cu", "sal_decode_ops.cu", "sal_pack.cu")]
HDRS = [os.path.join(REPO_DIR, "include", name) for name in ("sal_lutgemm.h", "sal_decode_ops.h", "sal_pack.h")]
LIB = os.path.join(PKG_DIR, "libsal_lutgemm.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
    "-cudart", "static",
    "--threads", "0",   # the three translation units compile side by side
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def up_to_date() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(p) <= t for p in (*SRCS, *HDRS, os.path.abspath(__file__)))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    cmd = [find_nvcc(), *NVCC_FLAGS, "-I", os.path.join(REPO_DIR, "include"), "-o", LIB, *SRCS]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

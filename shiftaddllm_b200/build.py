"""Builds ``libsal_lutgemm.so`` (CUDA kernels + C ABI) for sm_100a, in-tree.

Usage: ``python -m shiftaddllm_b200.build [--force] [--verbose] [--measure]``.
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
    "-Xlinker", "-soname=libsal_lutgemm.so",   # the compiled `lutgemm` module links to the library by this name
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


def build(force: bool = False, verbose: bool = False, measure: bool = False) -> str:
    """``measure=True`` compiles ``libsal_lutgemm_measure.so`` instead: the same library with
    -DSAL_MEASURE, i.e. with the ``sal_debug_set`` hook and the switches that turn parts of the kernel
    off for timing.  Point ``SAL_LUTGEMM_LIBRARY`` at it to use it."""
    if measure:
        out = os.path.join(PKG_DIR, "libsal_lutgemm_measure.so")
        cmd = [find_nvcc(), *NVCC_FLAGS, "-DSAL_MEASURE", "-I", os.path.join(REPO_DIR, "include"), "-o", out, *SRCS]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
        return out
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


EXT_DIR = os.path.join(PKG_DIR, "ext")
EXT_SRC = os.path.join(PKG_DIR, "csrc", "lutgemm_ext.cpp")


def extension_path() -> str:
    import sysconfig

    return os.path.join(EXT_DIR, "lutgemm" + sysconfig.get_config_var("EXT_SUFFIX"))


def extension_up_to_date() -> bool:
    out = extension_path()
    return os.path.exists(out) and all(os.path.getmtime(p) <= os.path.getmtime(out) for p in (EXT_SRC, HDRS[0], os.path.abspath(__file__)))


def build_extension(force: bool = False) -> str:
    """Compiles the `lutgemm` Python extension module (pybind11 + torch tensors over the C ABI) into
    ``shiftaddllm_b200/ext/``: what lut_gemm/setup_lut.py produces for the reference.  Plain g++; needs
    the torch and Python headers of the running interpreter.  The module finds ``libsal_lutgemm.so`` next
    to the package through its run path."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    if not os.path.exists(LIB):
        build()
    out = extension_path()
    if not force and extension_up_to_date():
        return out
    os.makedirs(EXT_DIR, exist_ok=True)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = cpp_extension.CUDA_HOME or "/usr/local/cuda"
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=lutgemm",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I", os.path.join(REPO_DIR, "include"), "-I", sysconfig.get_paths()["include"], "-I", os.path.join(cuda_home, "include")]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-o", out, EXT_SRC, LIB, "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath,$ORIGIN/..", f"-Wl,-rpath,{torch_lib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"g++ failed with exit code {res.returncode}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, measure="--measure" in sys.argv))
    if "--measure" not in sys.argv:
        print(build_extension(force="--force" in sys.argv))

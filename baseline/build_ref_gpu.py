"""Builds the timing harness around the reference's own CUDA kernel into the git-ignored ``baseline/_ref/``.

    python baseline/build_ref_gpu.py [reference_root]

The harness (``baseline/ref_lutgemm_bench.cu``, this repository's code) includes the reference's
``lut_gemm/mv_fp16_bias.hpp`` from where it lies in the reference tree; no reference source is copied.
Where the reference tree is absent the script does nothing and says so (the binary built earlier, if any,
is what ``bench.py`` runs).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def build(reference_root="/root/reference"):
    header_dir = os.path.join(reference_root, "lut_gemm")
    if not os.path.exists(os.path.join(header_dir, "mv_fp16_bias.hpp")):
        print(f"reference sources not found under {reference_root}: nothing built")
        return None
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "ref_lutgemm_bench")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-cudart", "static", "-w",
           "-I", header_dir, "-o", out, os.path.join(HERE, "ref_lutgemm_bench.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
    return out


if __name__ == "__main__":
    print(build(*sys.argv[1:2]))

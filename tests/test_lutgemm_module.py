"""The compiled `lutgemm` extension module (what lut_gemm/setup_lut.py builds for the reference) and the
reference-side call chain through it: ``import lutgemm`` -> ``LutLinear.forward`` (lut_gemm/quant.py:41-54)."""
import importlib
import os
import sys
import types

import numpy as np
import pytest
import torch

from oracle import bcq_oracle as o
from shiftaddllm_b200 import build, lutgemm as shim

REFERENCE = "/root/reference"
FIVE = ("lutgemm_compute", "lutgemm_compute_shift_scale", "lutgemm_compute_block", "lutgemm_compute_block_shift",
        "lutgemm_compute_block_shiftInt8")


@pytest.fixture(scope="module")
def module(lib):
    build.build_extension()
    saved = sys.modules.get("lutgemm")
    mod = shim.install()                     # registers the compiled module as `lutgemm`
    yield mod
    if saved is not None:
        sys.modules["lutgemm"] = saved
    else:
        sys.modules.pop("lutgemm", None)


def test_compiled_module_exports_the_reference_names(module):
    import lutgemm

    assert lutgemm is module and lutgemm.__file__.endswith(".so")
    for name in FIVE:
        assert callable(getattr(lutgemm, name)), name
    assert lutgemm.sal_version() == 100
    # no CPU path: a CPU tensor is refused with an error, nothing is computed on the host
    z16, z32 = torch.zeros(8, dtype=torch.float16), torch.zeros(8, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        lutgemm.lutgemm_compute_shift_scale(z16, z32, z16, torch.zeros(32, dtype=torch.float16), 8, 32, 1, 1)
    # the ctypes module offers the same names
    assert shim.install(compiled=False) is shim and all(hasattr(shim, n) for n in FIVE)
    shim.install()


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="the reference sources are not on this machine")
def test_reference_lutlinear_imports_with_this_module_installed(module):
    """The unmodified reference module lut_gemm/quant.py does `import lutgemm` at import time
    (lut_gemm/quant.py:5); with this build installed it imports and constructs its LutLinear."""
    sys.path.insert(0, REFERENCE)
    try:
        for name in [n for n in sys.modules if n == "lut_gemm" or n.startswith("lut_gemm.")]:
            del sys.modules[name]
        pkg = types.ModuleType("lut_gemm")           # the reference's package __init__ pulls in more than this path
        pkg.__path__ = [os.path.join(REFERENCE, "lut_gemm")]
        sys.modules["lut_gemm"] = pkg
        ref_quant = importlib.import_module("lut_gemm.quant")
        assert ref_quant.lutgemm is module
        lin = ref_quant.LutLinear(256, 64, 128, 3, bias=torch.zeros(64))
        assert tuple(lin.binaryWeight.shape) == (8, 3, 64) and lin.num_groups == 2
    finally:
        sys.path.remove(REFERENCE)
        for name in [n for n in sys.modules if n == "lut_gemm" or n.startswith("lut_gemm.")]:
            del sys.modules[name]


@pytest.mark.gpu
def test_literal_reference_forward_call(module):
    """The exact statements of the reference's forward (lut_gemm/quant.py:46-51): output = bias.clone();
    lutgemm.lutgemm_compute_block_shiftInt8(output, bW, alpha, x, N, K, wbit, num_groups, 3)."""
    import lutgemm

    k, n, q, gs = 1024, 512, 3, 16
    rng = np.random.default_rng(5)
    bw = rng.integers(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=np.int64).astype(np.int32)
    shifts = rng.integers(-9, -1, (k // 8, q, n // gs, 3)).astype(np.int8)
    shifts[::2, :, :, 2] = o.APOT_NONE
    x = rng.standard_normal((1, k)).astype(np.float16)
    bias = (0.02 * rng.standard_normal(n)).astype(np.float16)
    ref = o.lutgemm_compute_block_shift_int8(bias.astype(np.float32)[None, :], bw, shifts, x)
    t = lambda a: torch.from_numpy(a).cuda()
    output = t(bias).clone()
    lutgemm.lutgemm_compute_block_shiftInt8(output, t(bw), t(shifts), t(x), n, k, q, n // gs, 3)
    torch.cuda.synchronize()
    assert o.max_rel_err(output.float().cpu().numpy(), ref[0]) <= 1e-2
    # mode A through the compiled module, on a non-default stream, accumulate contract
    from shiftaddllm_b200 import synth

    layer = synth.make_layer(2048, 1024, 3, 128, packed_draw=True, bias=True)
    w = o.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
    want = o.linear_fp32(layer.x.numpy(), w, layer.bias.numpy())
    d = layer.to("cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        out = d.bias.clone()
        lutgemm.lutgemm_compute_shift_scale(out, d.bWeight, d.alpha, d.x, layer.N, layer.K, 3, layer.K // 128)
        y = torch.empty(1, layer.N, dtype=torch.float16, device="cuda")
        lutgemm.lutgemv_fused(y, d.bWeight, d.alpha, d.bias, d.x, layer.N, layer.K, 3, layer.K // 128, pdl=True)
    stream.synchronize()
    assert o.max_rel_err(out.float().cpu().numpy(), want[0]) <= 1e-2
    assert o.max_rel_err(y.float().cpu().numpy(), want) <= 1e-2


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="the reference sources are not on this machine")
def test_reference_lutlinear_forward_runs_on_this_build(module):
    """The reference's own LutLinear.forward, unmodified, on this build's kernels (square layer, int8 shifts
    written by hand: the reference's quantize_to_apot drops residual signs and emits 2**0 for exact powers of two)."""
    sys.path.insert(0, REFERENCE)
    try:
        pkg = types.ModuleType("lut_gemm")
        pkg.__path__ = [os.path.join(REFERENCE, "lut_gemm")]
        sys.modules["lut_gemm"] = pkg
        ref_quant = importlib.import_module("lut_gemm.quant")
        k = n = 512
        rng = np.random.default_rng(9)
        lin = ref_quant.LutLinear(k, n, 128, 3, bias=torch.from_numpy((0.02 * rng.standard_normal(n)).astype(np.float16)))
        bw = rng.integers(-2 ** 31, 2 ** 31, (k // 32, 3, n), dtype=np.int64).astype(np.int32)
        shifts = rng.integers(-9, -1, (k // 8, 3, n // 16, 3)).astype(np.int8)
        lin.binaryWeight = torch.from_numpy(bw)
        lin.alpha = torch.from_numpy(shifts)
        lin.num_groups = n // 16                       # what the reference's loader sets for block layouts
        lin = lin.cuda()
        lin.bias = lin.bias.cuda()
        x = torch.from_numpy(rng.standard_normal((1, k)).astype(np.float16)).cuda()
        y = lin(x)
        torch.cuda.synchronize()
        ref = o.lutgemm_compute_block_shift_int8(lin.bias.float().cpu().numpy()[None, :], bw, shifts, x.cpu().numpy())
        assert o.max_rel_err(y.float().cpu().numpy(), ref) <= 1e-2
    finally:
        sys.path.remove(REFERENCE)
        for name in [n_ for n_ in sys.modules if n_ == "lut_gemm" or n_.startswith("lut_gemm.")]:
            del sys.modules[name]

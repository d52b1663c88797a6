"""The C-ABI shared library: it loads, exports every symbol the header declares,
plans launches and validates arguments without needing a GPU."""
import ctypes
import os
import re

import pytest

from shiftaddllm_b200 import _lib

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = set()
    for header in ("sal_lutgemm.h", "sal_decode_ops.h", "sal_pack.h"):
        text = open(os.path.join(REPO, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"#ifdef SAL_MEASURE.*?#endif", "", text, flags=re.S)   # declared for measurement builds only
        names |= set(re.findall(r"\b(sal_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_exports_every_declared_symbol(lib):
    names = declared_functions()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/sal_lutgemm.h but not exported"
    # and the ctypes table covers exactly the header
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_strings(lib):
    assert lib.sal_version() == 100
    assert _lib.status_string(0) == "ok"
    assert "workspace" in _lib.status_string(_lib.SAL_E_WORKSPACE)
    assert lib.sal_workspace_bytes(1, 4096) == 16384 + 4096 * 64 * 4


def test_planner_without_gpu(lib):
    info = _lib.SalPlanInfo()
    assert lib.sal_plan_shift_scale(1, 4096, 4096, 3, 32, ctypes.byref(info)) == 0
    assert info.tiled == 1 and 1 <= info.ctas <= info.ranges * info.splits and info.stages >= 2
    assert info.smem_bytes <= 115712            # two CTAs must fit one SM
    assert lib.sal_plan_shift_scale(1, 4096, 4096, 3, 128, ctypes.byref(info)) == 0   # g = 32
    assert info.tiled == 0
    assert lib.sal_plan_shift_scale(4, 4096, 4096, 3, 32, ctypes.byref(info)) == 0    # small batch: half2-table variant
    assert info.tiled == 1
    assert lib.sal_plan_shift_scale(4, 4096, 4096, 5, 32, ctypes.byref(info)) == 0    # q > 4: generic kernel
    assert info.tiled == 0
    assert lib.sal_plan_shift_scale(1, 100, 64, 3, 1, ctypes.byref(info)) == _lib.SAL_E_SHAPE
    for k, n, q in ((4096, 11008, 3), (11008, 4096, 3), (8192, 28672, 2), (28672, 8192, 2), (8192, 1024, 2), (768, 768, 3)):
        assert lib.sal_plan_shift_scale(1, k, n, q, k // 128, ctypes.byref(info)) == 0
        assert info.tiled == 1 and 1 <= info.splits <= 64 and info.ctas >= 1


def test_argument_validation_happens_before_any_gpu_work(lib):
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 15) & ~15
    call = lib.sal_lutgemv_shift_scale
    assert call(None, p, None, p, p, 1, 256, 64, 3, 2, 0, None, 0, None) == _lib.SAL_E_NULL
    assert call(p, p, None, p, p, 1, 250, 64, 3, 2, 0, None, 0, None) == _lib.SAL_E_SHAPE      # K % 32
    assert call(p, p, None, p, p, 1, 256, 64, 9, 2, 0, None, 0, None) == _lib.SAL_E_SHAPE      # q > 8
    assert call(p, p, None, p, p, 65, 256, 64, 3, 2, 0, None, 0, None) == _lib.SAL_E_SHAPE     # M > 64
    assert call(p, p, None, p, p, 1, 256, 64, 3, 3, 0, None, 0, None) == _lib.SAL_E_SHAPE      # K % groups
    assert call(p + 2, p, None, p, p, 1, 256, 64, 3, 2, 0, None, 0, None) == _lib.SAL_E_ALIGN
    assert lib.sal_lutgemm_block(p, p, None, p, p, 1, 256, 64, 3, 5, 0, None, 0, None) == _lib.SAL_E_SHAPE  # N % groups
    assert lib.sal_lutgemv_grouped(None, 1, 0, None, 0, None) == _lib.SAL_E_NULL
    probs = (_lib.SalProblem * 1)()
    assert lib.sal_lutgemv_grouped(probs, 0, 0, None, 0, None) == _lib.SAL_E_SHAPE
    assert lib.sal_lutgemv_grouped(probs, 9, 0, None, 0, None) == _lib.SAL_E_SHAPE
    assert lib.sal_prepare_grouped(None, 1, 0, None, ctypes.byref(ctypes.c_void_p())) == _lib.SAL_E_NULL
    assert lib.sal_launch_prepared(None, None, 0, -1, None) == _lib.SAL_E_NULL
    assert lib.sal_prepared_workspace_bytes(None) == 0


def test_measurement_hook_is_not_in_the_product_library(lib):
    """The switches that turn parts of the kernel off for timing exist only in -DSAL_MEASURE builds."""
    assert not hasattr(lib, "sal_debug_set")


def test_no_cpu_fallback(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    buf = ctypes.create_string_buffer(1 << 16)
    p = (ctypes.addressof(buf) + 255) & ~255
    # well-formed arguments, but no device: the library must refuse, not compute on the host
    rc = lib.sal_lutgemv_shift_scale(p, p, None, p, p, 1, 256, 64, 3, 2, 0, None, 0, None)
    assert rc == _lib.SAL_E_DEVICE
    assert lib.sal_device_ok() == _lib.SAL_E_DEVICE


def test_planner_invariants_over_many_shapes(lib):
    """The work split of the tiled kernel, queried without a GPU for a grid of shapes: every CTA gets at least one unit
    (splits never exceed the units of a range), the K splits stay within the scratch layout, the ring has a slot per
    plane group, and the CTA's shared memory lets two CTAs share an SM."""
    info = _lib.SalPlanInfo()
    seen_tiled = 0
    for k in (256, 512, 768, 1024, 4096, 5120, 8192, 11008, 14336, 28672):
        for n in (8, 256, 264, 768, 1000, 4096, 11008, 32000):
            for q in (1, 2, 3, 4):
                for m in (1, 2, 7, 16, 64):
                    if k % 128:
                        continue
                    rc = lib.sal_plan_shift_scale(m, k, n, q, k // 128, ctypes.byref(info))
                    assert rc == 0, (m, k, n, q, rc)
                    if not info.tiled:
                        assert info.ctas >= 1
                        continue
                    seen_tiled += 1
                    tiles = (n + 255) // 256
                    assert 1 <= info.ranges <= tiles
                    assert 1 <= info.splits <= 64
                    units_per_range = -(-tiles // info.ranges) * (k // 256)      # upper bound for the widest range
                    assert info.splits <= units_per_range
                    assert info.ctas >= info.ranges
                    assert info.stages >= (2 if q == 4 else 1)
                    assert info.smem_bytes <= 115712
    assert seen_tiled > 500

"""The entry point that brings its own scratch (``sal_lutgemv_shift_scale_static``).

Some hosts may not allocate device memory once they are up — an inference server whose pool owns
the GPU, code running inside another component's stream capture — so this entry keeps the split-K
scratch in a fixed array inside the library.  The test drives it through the C ABI, twice in a row
(the second call meets the first call's leftovers in the shared array), and compares with the
ordinary entry point that takes a caller-allocated workspace.  Collected last on purpose: a run that
stops at the first failure has then already run everything else.
"""
import numpy as np
import pytest
import torch

from oracle import bcq_oracle as o
from shiftaddllm_b200 import _lib, lutgemm, synth

pytestmark = pytest.mark.gpu
TOL = 1e-2   # same bar as tests/test_gpu_parity.py: max|y - y_ref| / max|y_ref|


def _call_static(lib, layer, d, y, flags=0):
    return lib.sal_lutgemv_shift_scale_static(d.bWeight.data_ptr(), d.alpha.data_ptr(),
                                              d.bias.data_ptr() if d.bias is not None else None, d.x.data_ptr(),
                                              y.data_ptr(), 1, layer.K, layer.N, layer.q, layer.K // layer.g, flags,
                                              torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_workspace_entry_twice():
    lib = _lib.load()
    # 4096x4096 q3 splits K sixteen ways: the scratch array is really used
    info = _lib.SalPlanInfo()
    assert lib.sal_plan_shift_scale(1, 4096, 4096, 3, 32, info) == 0 and info.tiled == 1 and info.splits > 1
    layers = [synth.make_layer(4096, 4096, 3, 128, packed_draw=True, layer_index=5),
              synth.make_layer(2048, 1024, 2, 128, packed_draw=True, bias=True, layer_index=6)]
    for rep in range(2):                       # two calls in a row per shape, interleaved shapes
        for layer in layers:
            d = layer.to("cuda")
            y_ws = torch.empty(1, layer.N, dtype=torch.float16, device="cuda")
            lutgemm.lutgemv_fused(y_ws, d.bWeight, d.alpha, d.bias, d.x, layer.N, layer.K, layer.q, layer.K // layer.g)
            y_st = torch.full((1, layer.N), float("nan"), dtype=torch.float16, device="cuda")
            assert _call_static(lib, layer, d, y_st) == 0
            torch.cuda.synchronize()
            a, b = y_st.float().cpu().numpy(), y_ws.float().cpu().numpy()
            assert np.isfinite(a).all()
            assert o.max_rel_err(a, b) <= TOL
            assert np.array_equal(a, b)        # same kernel, same fixed reduction order
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sal_static_status(stream) == 0          # no bounded wait expired, no unsupported variant ran
    # the contract itself: after the first call on the device, a call takes no device memory at all
    layer, d = layers[0], layers[0].to("cuda")
    y_st = torch.empty(1, layer.N, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = torch.cuda.memory_allocated()
    for _ in range(3):
        assert _call_static(lib, layer, d, y_st) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == torch_before
    assert lib.sal_static_status(stream) == 0
    layer = layers[1]
    a = None
    d = layer.to("cuda")
    y_st = torch.empty(1, layer.N, dtype=torch.float16, device="cuda")
    assert _call_static(lib, layer, d, y_st) == 0
    torch.cuda.synchronize()
    a = y_st.float().cpu().numpy()
    # and against the oracle once, so that both being wrong together cannot pass
    layer = layers[1]
    w = o.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
    ref = o.linear_fp32(layer.x.numpy(), w, layer.bias.numpy())
    assert o.max_rel_err(a, ref) <= TOL


def test_static_scratch_rejects_oversize():
    lib = _lib.load()
    layer = synth.make_layer(256, 64, 3, 128)
    d = layer.to("cuda")
    y = torch.empty(1, 64, dtype=torch.float16, device="cuda")
    # N beyond the built-in scratch: refused with the workspace error before anything is launched
    rc = lib.sal_lutgemv_shift_scale_static(d.bWeight.data_ptr(), d.alpha.data_ptr(), None, d.x.data_ptr(),
                                            y.data_ptr(), 1, 256, 16384 + 8, 3, 2, 0,
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.SAL_E_WORKSPACE
    assert "workspace" in _lib.status_string(rc)

"""Parity of the CUDA path (called through the C ABI) with the oracle.

Floating-point bar: ``max|y - y_ref| / max|y_ref| <= 1e-2`` against the
dequantise-then-matmul oracle evaluated in fp32 (the tolerance the task states
for fp16 accumulation; the kernels accumulate in fp32 and land near 5e-4, the
rounding of the fp16 output).  Integer work (packing) is bit-exact and is
covered by the CPU tests.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import bcq_oracle as o
from shiftaddllm_b200 import _lib, lutgemm, synth
from shiftaddllm_b200.quant import LutLinear

pytestmark = pytest.mark.gpu
TOL = 1e-2


def dev(t):
    return None if t is None else t.cuda()


def ref_mode_a(layer):
    w = o.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
    return o.linear_fp32(layer.x.numpy(), w, None if layer.bias is None else layer.bias.numpy())


def run_mode_a(layer, *, pdl=False):
    m = layer.x.shape[0]
    y = torch.empty(m, layer.N, dtype=torch.float16, device="cuda")
    lutgemm.lutgemv_fused(y, dev(layer.bWeight), dev(layer.alpha), dev(layer.bias), dev(layer.x), layer.N, layer.K,
                          layer.q, layer.K // layer.g, pdl=pdl)
    torch.cuda.synchronize()
    return y.float().cpu().numpy()


def assert_status_clean():
    lib = _lib.load()
    ws = lutgemm.workspace_for(torch.device("cuda", torch.cuda.current_device()), 1, 8)
    assert lib.sal_workspace_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0


def test_library_loaded_and_device_ok(lib):
    assert lib.sal_device_ok() == 0


def test_golden_layer(golden):
    """The layer whose inputs AND output were produced by the reference's own Python."""
    bw = torch.from_numpy(o.to_kernel_layout(golden["la_packed"])).cuda()
    alpha = torch.from_numpy(np.ascontiguousarray(np.transpose(golden["la_alpha_f16"], (1, 2, 0)))).cuda()
    x = torch.from_numpy(golden["la_x_f16"]).cuda()
    bias = torch.from_numpy(golden["la_bias_f16"]).cuda()
    n, k = bw.shape[2], bw.shape[0] * 32
    # reference contract: output pre-loaded with the bias, kernel accumulates (lut_gemm/quant.py:46-51)
    out = bias.clone()
    lutgemm.lutgemm_compute_shift_scale(out, bw, alpha, x, n, k, 3, alpha.shape[0])
    torch.cuda.synchronize()
    assert o.max_rel_err(out.float().cpu().numpy(), golden["la_y"][0]) <= TOL
    # fused-bias variant gives the same numbers
    y = torch.empty(1, n, dtype=torch.float16, device="cuda")
    lutgemm.lutgemv_fused(y, bw, alpha, bias, x, n, k, 3, alpha.shape[0])
    torch.cuda.synchronize()
    assert o.max_rel_err(y.float().cpu().numpy()[0], golden["la_y"][0]) <= TOL


def test_config1_opt125m_qproj():
    layer = synth.make_layer(768, 768, 3, 128, bias=True)
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL
    assert_status_clean()


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 11008), (11008, 4096)])
def test_config2_llama7b_shapes(k, n):
    layer = synth.make_layer(k, n, 3, 128, packed_draw=True, layer_index=k % 97)
    ref = ref_mode_a(layer)
    assert o.max_rel_err(run_mode_a(layer), ref) <= TOL
    assert o.max_rel_err(run_mode_a(layer, pdl=True), ref) <= TOL
    assert_status_clean()


@pytest.mark.parametrize("q", [1, 2, 3, 4, 5])
def test_bit_widths(q):
    layer = synth.make_layer(1024, 512, q, 128, packed_draw=True)
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL


@pytest.mark.parametrize("k,n,g", [(2048, 1024, 256), (2048, 1024, 2048), (1024, 1376, 128), (512, 264, 128),
                                   (256, 8, 128), (8192, 1024, 128)])
def test_group_sizes_and_column_tails(k, n, g):
    layer = synth.make_layer(k, n, 2, g, packed_draw=True)
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL
    assert_status_clean()


@pytest.mark.parametrize("k,n,g", [(96, 30, 32), (160, 66, 32), (320, 100, 64), (64, 2, 64), (32, 1, 32)])
def test_generic_kernel_odd_shapes(k, n, g):
    """Shapes the tiled kernel does not take (K % 256, N % 8, small groups) — the reference's
    own limits are K % 32 == 0 and N even."""
    layer = synth.make_layer(k, n, 3, g, bias=True)
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL


@pytest.mark.parametrize("m", [1, 4, 8, 16, 64])
def test_config3_small_batch(m):
    for q in (2, 3, 4):
        layer = synth.make_layer(1024, 768, q, 128, M=m, packed_draw=True, layer_index=m)
        assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL


def test_tiled_and_generic_kernels_agree():
    layer = synth.make_layer(1024, 1024, 3, 128, packed_draw=True)
    y_tiled = run_mode_a(layer)
    lib = _lib.load()
    y = torch.zeros(1, layer.N, dtype=torch.float16, device="cuda")
    bw, al, x = dev(layer.bWeight), dev(layer.alpha), dev(layer.x)
    rc = lib.sal_lutgemv_shift_scale(bw.data_ptr(), al.data_ptr(), None, x.data_ptr(), y.data_ptr(), 1, layer.K,
                                     layer.N, layer.q, layer.K // layer.g, _lib.SAL_FORCE_GENERIC, None, 0,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert o.max_rel_err(y.float().cpu().numpy(), y_tiled) <= 2e-3   # both round an fp32 sum to fp16


def test_deterministic_and_workspace_reusable():
    layer = synth.make_layer(4096, 4096, 3, 128, packed_draw=True)
    a = run_mode_a(layer)
    for _ in range(3):
        assert np.array_equal(run_mode_a(layer), a)   # fixed reduction order: bit-identical every time


def test_accumulate_semantics():
    layer = synth.make_layer(1024, 512, 3, 128, packed_draw=True)
    base = torch.randn(1, 512, generator=torch.Generator().manual_seed(1)).half()
    out = base.clone().cuda()
    lutgemm.lutgemm_compute_shift_scale(out, dev(layer.bWeight), dev(layer.alpha), dev(layer.x), 512, 1024, 3, 8)
    torch.cuda.synchronize()
    ref = ref_mode_a(layer) + base.float().numpy()
    assert o.max_rel_err(out.float().cpu().numpy(), ref) <= TOL


def test_without_workspace_no_split():
    """A NULL workspace is legal: the planner then keeps K in one piece."""
    lib = _lib.load()
    layer = synth.make_layer(2048, 512, 3, 128, packed_draw=True)
    bw, al, x = dev(layer.bWeight), dev(layer.alpha), dev(layer.x)
    y = torch.empty(1, 512, dtype=torch.float16, device="cuda")
    rc = lib.sal_lutgemv_shift_scale(bw.data_ptr(), al.data_ptr(), None, x.data_ptr(), y.data_ptr(), 1, 2048, 512, 3,
                                     16, 0, None, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert o.max_rel_err(y.float().cpu().numpy(), ref_mode_a(layer)) <= TOL


def test_grouped_launch_qkv():
    layers = [synth.make_layer(4096, n, 3, 128, packed_draw=True, layer_index=i, bias=(i == 1))
              for i, n in enumerate((4096, 1024, 1024))]
    probs, outs = [], []
    for layer in layers:
        y = torch.empty(1, layer.N, dtype=torch.float16, device="cuda")
        outs.append(y)
        probs.append(dict(output=y, bWeight=dev(layer.bWeight), alpha=dev(layer.alpha), bias=dev(layer.bias),
                          d_input=dev(layer.x), mSize=layer.N, kSize=layer.K, nb=3, num_groups=32))
    lutgemm.lutgemv_grouped(probs, pdl=True)
    torch.cuda.synchronize()
    for layer, y in zip(layers, outs):
        assert o.max_rel_err(y.float().cpu().numpy(), ref_mode_a(layer)) <= TOL
    assert_status_clean()


def test_fused_swiglu_input():
    """down_proj with x = silu(gate) * up formed inside the table build equals the two-step path."""
    import torch.nn.functional as F

    from shiftaddllm_b200 import decode_ops

    for m in (1, 3):
        layer = synth.make_layer(2048, 512, 3, 128, M=m, packed_draw=True)
        g = torch.Generator().manual_seed(9)
        gate, up = torch.randn(m, 2048, generator=g).half().cuda(), torch.randn(m, 2048, generator=g).half().cuda()
        bw, al = dev(layer.bWeight), dev(layer.alpha)
        y_fused = torch.empty(m, 512, dtype=torch.float16, device="cuda")
        lutgemm.lutgemv_grouped([dict(output=y_fused, bWeight=bw, alpha=al, bias=None, d_input=gate, d_input_mul=up,
                                      mSize=512, kSize=2048, nb=3, num_groups=16)])
        act = torch.empty_like(gate)
        decode_ops.silu_mul(gate, up, act)
        y_two = torch.empty_like(y_fused)
        lutgemm.lutgemv_grouped([dict(output=y_two, bWeight=bw, alpha=al, bias=None, d_input=act, mSize=512, kSize=2048,
                                      nb=3, num_groups=16)])
        torch.cuda.synchronize()
        assert torch.equal(y_fused, y_two)
        w = o.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
        ref = o.linear_fp32((F.silu(gate.float()) * up.float()).cpu().numpy(), w)
        assert o.max_rel_err(y_fused.float().cpu().numpy(), ref) <= TOL


FIXED_ONE = float(2 ** 32)   # a fixed-point accumulator counts units of 2**-32


@pytest.mark.parametrize("k,n", [(768, 768), (4096, 4096), (11008, 4096)])
def test_fixed_point_atomic_output(k, n):
    """Opt-in accumulator output (int64, units of 2**-32) that every K split adds its partial sum to with integer
    atomics (bias added once): tighter than the fp16 output because nothing is rounded to fp16, it accumulates
    onto what the buffer held, and — integer sums not depending on the order of arrival — it is bit-identical
    from call to call."""
    layer = synth.make_layer(k, n, 3, 128, packed_draw=True, bias=True, layer_index=5)
    ref = ref_mode_a(layer)
    base = torch.randn(1, n, generator=torch.Generator().manual_seed(2)).cuda()
    base_fixed = torch.round(base.double() * FIXED_ONE).to(torch.int64)
    prob = dict(bWeight=dev(layer.bWeight), alpha=dev(layer.alpha), bias=dev(layer.bias), d_input=dev(layer.x), mSize=n, kSize=k,
                nb=3, num_groups=k // 128)
    results = []
    for _ in range(3):
        y = base_fixed.clone()
        lutgemm.lutgemv_grouped([dict(output=y, **prob)], atomic_fixed=True)
        torch.cuda.synchronize()
        results.append(y)
    got = ((results[0] - base_fixed).double() / FIXED_ONE).cpu().numpy()
    assert o.max_rel_err(got, ref) <= 1e-4
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])      # deterministic
    assert_status_clean()
    # refused where the fixed-order reduction is the only implementation: M > 1
    lib = _lib.load()
    x2 = torch.zeros(2, k, dtype=torch.float16, device="cuda")
    y2 = torch.zeros(2, n, dtype=torch.int64, device="cuda")
    rc = lib.sal_lutgemv_shift_scale(prob["bWeight"].data_ptr(), prob["alpha"].data_ptr(), None, x2.data_ptr(),
                                     y2.data_ptr(), 2, k, n, 3, k // 128, _lib.SAL_OUT_FIXED_ATOMIC, None, 0,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.SAL_E_UNSUPPORTED


def test_fixed_point_swiglu_input():
    """down projection reading fixed-point gate/up accumulators and adding into a fixed-point output."""
    import torch.nn.functional as F

    layer = synth.make_layer(2048, 512, 3, 128, packed_draw=True)
    g = torch.Generator().manual_seed(11)
    gate, up = torch.randn(1, 2048, generator=g).cuda(), torch.randn(1, 2048, generator=g).cuda()
    gate_fixed = torch.round(gate.double() * FIXED_ONE).to(torch.int64)
    up_fixed = torch.round(up.double() * FIXED_ONE).to(torch.int64)
    y = torch.zeros(1, 512, dtype=torch.int64, device="cuda")
    lutgemm.lutgemv_grouped([dict(output=y, bWeight=dev(layer.bWeight), alpha=dev(layer.alpha), bias=None, d_input=gate_fixed,
                                  d_input_mul=up_fixed, mSize=512, kSize=2048, nb=3, num_groups=16)],
                            atomic_fixed=True, swiglu_fixed=True)
    torch.cuda.synchronize()
    w = o.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
    act = (F.silu(gate.half().float()).half().float() * up.half().float()).half().float()   # rounded to fp16 at every step, as the table build does
    assert o.max_rel_err((y.double() / FIXED_ONE).cpu().numpy(), o.linear_fp32(act.cpu().numpy(), w)) <= 2e-3


def test_hand_checkable():
    k, n, q = 512, 256, 2
    bw = torch.full((k // 32, q, n), -1, dtype=torch.int32, device="cuda")          # every bit set: all +1
    alpha = torch.full((k // 128, q, n), 0.25, dtype=torch.float16, device="cuda")
    x = torch.arange(k, dtype=torch.float32).mul(1 / 64).half().cuda()
    y = torch.empty(1, n, dtype=torch.float16, device="cuda")
    lutgemm.lutgemv_fused(y, bw, alpha, None, x.view(1, -1), n, k, q, k // 128)
    expect = q * 0.25 * x.float().sum().item()
    assert torch.allclose(y.float(), torch.full_like(y, expect, dtype=torch.float32), rtol=2e-3)
    bw.zero_()                                                                        # all -1
    lutgemm.lutgemv_fused(y, bw, alpha, None, x.view(1, -1), n, k, q, k // 128)
    assert torch.allclose(y.float(), torch.full_like(y, -expect, dtype=torch.float32), rtol=2e-3)
    # one-hot activation: y[n] = x_k * sum_b alpha * sign_b(k, n)
    layer = synth.make_layer(512, 256, 3, 128, packed_draw=True)
    x1 = torch.zeros(1, 512, dtype=torch.float16)
    x1[0, 300] = 1.5
    layer.x = x1
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL


def test_other_entry_points():
    rng = np.random.default_rng(7)
    k, n, q, m = 512, 192, 3, 3
    bw_np = rng.integers(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=np.int64).astype(np.int32)
    x_np = rng.standard_normal((m, k)).astype(np.float16)
    bw, x = torch.from_numpy(bw_np).cuda(), torch.from_numpy(x_np).cuda()
    # lutgemm_compute: one alpha per group halved per plane + q_bias
    a_np = rng.random((k // 128, n)).astype(np.float16)
    qb_np = (0.05 * rng.standard_normal((k // 128, n))).astype(np.float16)
    out = torch.zeros(1, n, dtype=torch.float16, device="cuda")
    lutgemm.lutgemm_compute(out, bw, torch.from_numpy(a_np).cuda(), torch.from_numpy(qb_np).cuda(), x[:1], n, k, q, k // 128)
    torch.cuda.synchronize()
    assert o.max_rel_err(out.float().cpu().numpy()[0], o.lutgemm_compute(np.zeros(n), bw_np, a_np, qb_np, x_np[0])) <= TOL
    # block (mode B) fp16
    ng = 12
    ab_np = rng.random((k // 8, q, ng)).astype(np.float16)
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    lutgemm.lutgemm_compute_block(out, bw, torch.from_numpy(ab_np).cuda(), x, n, k, q, ng)
    torch.cuda.synchronize()
    assert o.max_rel_err(out.float().cpu().numpy(), o.lutgemm_compute_block(np.zeros((m, n)), bw_np, ab_np, x_np)) <= TOL
    # block uint16 APoT (three 3-bit exponents)
    au_np = rng.integers(0, 512, (k // 8, q, ng)).astype(np.int16)
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    lutgemm.lutgemm_compute_block_shift(out, bw, torch.from_numpy(au_np).cuda(), x * 0.01, n, k, q, ng, 3)
    torch.cuda.synchronize()
    ref = o.lutgemm_compute_block_shift(np.zeros((m, n)), bw_np, au_np, (torch.from_numpy(x_np) * 0.01).numpy())
    assert o.max_rel_err(out.float().cpu().numpy(), ref) <= TOL
    # block int8 APoT, including explicit "no term"
    ai_np = rng.integers(-9, -1, (k // 8, q, ng, 3)).astype(np.int8)
    ai_np[::3, :, :, 2] = o.APOT_NONE
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    lutgemm.lutgemm_compute_block_shiftInt8(out, bw, torch.from_numpy(ai_np).cuda(), x, n, k, q, ng, 3)
    torch.cuda.synchronize()
    ref = o.lutgemm_compute_block_shift_int8(np.zeros((m, n)), bw_np, ai_np, x_np)
    assert o.max_rel_err(out.float().cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("k,n,gs,q,m", [(1024, 512, 16, 3, 1), (2048, 1024, 32, 2, 1), (512, 768, 128, 4, 3),
                                         (1024, 1024, 256, 3, 1), (1024, 1024, 512, 3, 2), (768, 1376, 16, 3, 1),
                                         (4096, 4096, 16, 3, 1), (1024, 512, 64, 1, 5)])
def test_block_modes_on_the_tiled_kernel(k, n, gs, q, m):
    """Shapes the TMA-ring kernel takes in block mode (K % 256 == 0, gs a power of two >= 16 or a
    multiple of 256): all three multiplier encodings against the dequantise oracle, and against the
    generic kernel (same fp32 arithmetic, different summation order)."""
    rng = np.random.default_rng(k + n + gs)
    ng = n // gs
    bw_np = rng.integers(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=np.int64).astype(np.int32)
    x_np = rng.standard_normal((m, k)).astype(np.float16)
    bias_np = (0.02 * rng.standard_normal(n)).astype(np.float16)
    bw, x = torch.from_numpy(bw_np).cuda(), torch.from_numpy(x_np).cuda()
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream

    def both(entry, alpha, *extra, x=x):
        outs = []
        for flags in (0, _lib.SAL_FORCE_GENERIC):
            y = torch.from_numpy(np.tile(bias_np, (m, 1))).cuda()      # the reference contract: output pre-loaded, kernel adds
            ws = lutgemm.workspace_for(y.device, m, n)
            rc = getattr(lib, entry)(bw.data_ptr(), alpha.data_ptr(), None, x.data_ptr(), y.data_ptr(), m, k, n, q, ng, *extra,
                                     flags | _lib.SAL_ACCUMULATE, ws.data_ptr(), ws.numel() * ws.element_size(), stream)
            assert rc == 0
            torch.cuda.synchronize()
            outs.append(y.float().cpu().numpy())
        assert o.max_rel_err(outs[0], outs[1]) <= 2e-3
        return outs[0]

    def ref(mult, xr=x_np):   # mult: fp32 [K/8, q, ng]
        return o.linear_fp32(xr, o.dequant_mode_b(bw_np, mult), bias_np)

    a16 = np.exp2(-rng.integers(2, 9, (k // 8, q, ng))).astype(np.float16) * rng.choice([1.0, 1.5, -1.25], (k // 8, q, ng)).astype(np.float16)
    assert o.max_rel_err(both("sal_lutgemm_block", torch.from_numpy(a16).cuda()), ref(a16.astype(np.float32))) <= TOL
    au = rng.integers(0, 512, (k // 8, q, ng)).astype(np.int16)
    mult_u = (np.exp2(au & 7) + np.exp2((au >> 3) & 7) + np.exp2((au >> 6) & 7)).astype(np.float32)
    xs_np = (x_np.astype(np.float32) * 0.01).astype(np.float16)     # multipliers reach 384: keep y inside fp16
    assert o.max_rel_err(both("sal_lutgemm_block_shift", torch.from_numpy(au).cuda(), x=torch.from_numpy(xs_np).cuda()),
                         ref(mult_u, xs_np)) <= TOL
    ai = rng.integers(-9, -1, (k // 8, q, ng, 3)).astype(np.int8)
    ai[::3, :, :, 2] = o.APOT_NONE
    mult_i = np.where(ai == o.APOT_NONE, 0.0, np.exp2(ai.astype(np.float32))).sum(-1).astype(np.float32)
    assert o.max_rel_err(both("sal_lutgemm_block_shift_int8", torch.from_numpy(ai).cuda(), 3), ref(mult_i)) <= TOL
    assert_status_clean()


def test_limits_of_the_interface():
    """The documented extremes: 8 bit planes (generic kernel), 64 activation rows in one call, the
    smallest legal K, and the first values past the limits (error codes, nothing launched)."""
    lib = _lib.load()
    layer = synth.make_layer(256, 64, 8, 128, bias=True)                       # q = SAL_MAX_Q
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL
    layer = synth.make_layer(512, 256, 2, 128, M=64, packed_draw=True)          # M = SAL_MAX_M
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL
    layer = synth.make_layer(32, 8, 3, 32)                                      # one packed word per column
    assert o.max_rel_err(run_mode_a(layer), ref_mode_a(layer)) <= TOL
    bw, al, x = dev(layer.bWeight), dev(layer.alpha), dev(layer.x)
    y = torch.zeros(1, 8, dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call(m, k, n, q, groups):
        return lib.sal_lutgemv_shift_scale(bw.data_ptr(), al.data_ptr(), None, x.data_ptr(), y.data_ptr(), m, k, n, q, groups, 0,
                                           None, 0, stream)

    assert call(65, 32, 8, 3, 1) == _lib.SAL_E_SHAPE        # too many rows
    assert call(1, 32, 8, 9, 1) == _lib.SAL_E_SHAPE         # too many planes
    assert call(1, 48, 8, 3, 1) == _lib.SAL_E_SHAPE         # K not a multiple of 32
    assert call(0, 32, 8, 3, 1) == _lib.SAL_E_SHAPE         # empty batch
    assert call(1, 32, 0, 3, 1) == _lib.SAL_E_SHAPE         # no output columns
    assert call(1, 32, 8, 3, 3) == _lib.SAL_E_SHAPE         # groups do not divide K
    torch.cuda.synchronize()
    assert not y.any()                                       # nothing ran


def test_bad_calls_raise():
    layer = synth.make_layer(256, 64, 3, 128)
    bw, al, x = dev(layer.bWeight), dev(layer.alpha), dev(layer.x)
    y = torch.empty(1, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        lutgemm.lutgemm_compute_shift_scale(y, bw, al, x.cpu(), 64, 256, 3, 2)           # CPU tensor
    with pytest.raises(RuntimeError):
        lutgemm.lutgemm_compute_shift_scale(y, bw, al.float(), x, 64, 256, 3, 2)         # wrong dtype
    with pytest.raises(RuntimeError):
        lutgemm.lutgemm_compute_shift_scale(y, bw, al, x, 64, 256, 3, 3)                 # alpha size mismatch
    with pytest.raises(RuntimeError):
        lutgemm.lutgemm_compute_shift_scale(y, bw[:, :2].contiguous(), al, x, 64, 256, 3, 2)  # bWeight size
    with pytest.raises(RuntimeError):
        lutgemm.lutgemm_compute_shift_scale(y, bw, al, x[:, :128].contiguous(), 64, 256, 3, 2)


def test_lutlinear_forward_modes():
    layer = synth.make_layer(1024, 512, 3, 128, M=5, bias=True, packed_draw=True)
    lin = LutLinear(1024, 512, 128, 3, bias=layer.bias.clone())
    lin.binaryWeight = layer.bWeight.clone()
    lin.set_row_alpha(layer.alpha)
    lin = lin.cuda()
    lin.bias = lin.bias.cuda()
    ref = ref_mode_a(layer)
    y = lin(layer.x.cuda().view(1, 5, 1024))
    assert y.shape == (1, 5, 512) and y.dtype == torch.float16
    assert o.max_rel_err(y.float().cpu().numpy()[0], ref) <= TOL
    y1 = lin(layer.x[:1].cuda())                                   # the reference's single-token case
    assert o.max_rel_err(y1.float().cpu().numpy(), ref[:1]) <= TOL
    # mode B through the literal int8 call of the reference's forward
    rng = np.random.default_rng(3)
    blk = np.exp2(-rng.integers(2, 9, (1024 // 8, 3, 512 // 16))).astype(np.float32)
    lin_b = LutLinear(1024, 512, 128, 3, bias=layer.bias.clone())
    lin_b.binaryWeight = layer.bWeight.clone()
    lin_b.set_block_alpha(torch.from_numpy(blk), apot=True)
    assert lin_b.alpha.dtype == torch.int8
    lin_b = lin_b.cuda()
    lin_b.bias = lin_b.bias.cuda()
    yb = lin_b(layer.x[:1].cuda())
    wb = o.dequant_mode_b(layer.bWeight.numpy(), blk)
    refb = o.linear_fp32(layer.x[:1].numpy(), wb, layer.bias.numpy())
    assert o.max_rel_err(yb.float().cpu().numpy(), refb) <= TOL


def test_full_size_properties():
    """Size-independent checks at the largest benchmark shapes, where the dequantise oracle
    would take minutes: negating x negates y; complementing every weight bit negates y;
    zero activations give exactly the bias."""
    k, n, q = 8192, 28672, 2
    gen = torch.Generator(device="cuda").manual_seed(0)
    bw = torch.randint(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=torch.int32, device="cuda", generator=gen)
    alpha = torch.exp2(-torch.randint(2, 9, (k // 128, q, n), device="cuda", generator=gen).float()).half()
    x = torch.randn(1, k, device="cuda", generator=gen).half()
    bias = (0.02 * torch.randn(n, device="cuda", generator=gen)).half()

    def run(bw_, x_, b_):
        y = torch.empty(1, n, dtype=torch.float16, device="cuda")
        lutgemm.lutgemv_fused(y, bw_, alpha, b_, x_, n, k, q, k // 128)
        return y

    y = run(bw, x, None)
    assert torch.equal(run(bw, -x, None), -y)
    assert torch.equal(run(~bw, x, None), -y)
    assert torch.equal(run(bw, torch.zeros_like(x), bias), bias.view(1, -1))
    assert float(y.float().abs().max()) > 1.0
    assert_status_clean()

"""The numpy/C oracle against the vectors produced by the reference's own Python
(tests/golden/make_golden.py) and against the reference's only self-check,
``unpack(pack(B), alpha) == einsum(B, alpha)``."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from oracle import bcq_oracle as o

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("tag", ["p0", "p1", "p2"])
def test_pack_bit_exact(golden, tag):
    packed = o.pack_binary_weight(golden[f"{tag}_planes"])
    assert packed.dtype == np.int32
    assert np.array_equal(packed, golden[f"{tag}_packed"])


@pytest.mark.parametrize("tag", ["p0", "p1", "p2"])
def test_unpack_bit_identical_and_roundtrip(golden, tag):
    w = o.unpack_weight(golden[f"{tag}_packed"], golden[f"{tag}_alpha"])
    assert np.array_equal(w, golden[f"{tag}_weight"])
    # the reference's self-check (zeroShot/models/kernel.py:96-120): prints max abs diff, expects 0
    assert np.max(np.abs(w - golden[f"{tag}_einsum"])) < 1e-5


@pytest.mark.parametrize("tag", ["p0", "p1", "p2"])
def test_fake_binary_weight(golden, tag):
    planes = golden[f"{tag}_planes"]
    fake = o.unpack_to_fake_binary_weight(golden[f"{tag}_packed"], planes.shape[1])
    assert np.array_equal(fake, planes)
    assert np.array_equal(fake.astype(np.uint8), golden[f"{tag}_fake_u8"])  # the reference returns uint8


def test_sign_bit_wraps_negative(golden):
    # p1 has element 31 of every row set in plane 0: the packed word must be negative as int32
    assert (golden["p1_packed"][:, 0, 0] < 0).all()
    assert np.array_equal(o.pack_binary_weight(golden["p1_planes"]), golden["p1_packed"])


def test_convert_weight_square(golden):
    bw, alpha = o.convert_weight(golden["cv_packed_lat"], np.repeat(golden["cv_alpha_blk"], 8, axis=0))
    assert np.array_equal(bw, golden["cv_kernel_bw"])
    assert np.array_equal(alpha, golden["cv_kernel_alpha"])


def test_convert_weight_nonsquare_matches_dequant():
    # the reference's convert_weight raises for non-square layers; the expectation is derived
    # from unpack_weight instead: both layouts must dequantise to the same matrix
    rng = np.random.default_rng(5)
    k_in, n_out, q, gs = 64, 96, 3, 16
    planes = rng.integers(0, 2, (k_in, n_out // gs, gs, q)).astype(np.int8) * 2 - 1
    packed_lat = o.pack_binary_weight(planes)
    alpha_blk = rng.random((k_in // 8, n_out // gs, q), dtype=np.float32) + 0.1
    w_t = o.unpack_weight(packed_lat, np.repeat(alpha_blk, 8, axis=0))  # [K, N]
    bw, alpha = o.convert_weight(packed_lat, alpha_blk)                 # [K/32,q,N], [K/8,q,N/gs]
    assert bw.shape == (k_in // 32, q, n_out)
    w = o.dequant_mode_b(bw, alpha)                                     # [N, K]
    assert np.array_equal(w, np.ascontiguousarray(w_t.T))


def test_apot_matches_reference(golden):
    assert np.array_equal(o.quantize_to_apot(golden["apot_in"]), golden["apot_out"])
    marked = o.quantize_to_apot(np.array([0.25, 2.0 ** -7], dtype=np.float32), mark_missing=True)
    assert marked.tolist() == [[-2, o.APOT_NONE, o.APOT_NONE], [-7, o.APOT_NONE, o.APOT_NONE]]
    assert np.allclose(o.apot_i8_multiplier(marked), [0.25, 2.0 ** -7])


def test_mode_a_layer_output(golden):
    bwk = o.to_kernel_layout(golden["la_packed"])
    ak = np.ascontiguousarray(np.transpose(golden["la_alpha_f16"], (1, 2, 0)))
    w = o.dequant_mode_a(bwk, ak)
    assert np.array_equal(w, golden["la_weight"])
    y = o.linear_fp32(golden["la_x_f16"], w, golden["la_bias_f16"])
    assert np.allclose(y, golden["la_y"], rtol=0, atol=2e-6)
    # the table-gather formulation agrees with dequantise-then-matmul (pins bit/byte conventions)
    y_lut = o.lut_gemv_mode_a(bwk, ak, golden["la_x_f16"]) + golden["la_bias_f16"].astype(np.float32)
    assert o.max_rel_err(y_lut, golden["la_y"][0]) < 1e-6


def test_hand_checkable_cases():
    k, n, q, g = 64, 8, 2, 32
    ones = np.ones((n, k // g, g, q), dtype=np.int8)
    bw = o.to_kernel_layout(o.pack_binary_weight(ones))
    alpha = np.full((k // g, q, n), 0.5, dtype=np.float32)
    x = np.arange(k, dtype=np.float32).astype(np.float16)
    y = o.lutgemm_compute_shift_scale(np.zeros(n, np.float32), bw, alpha, x)
    assert np.allclose(y, q * 0.5 * x.astype(np.float32).sum())
    # one-hot activation picks one weight column
    x1 = np.zeros(k, dtype=np.float16)
    x1[37] = 2.0
    rng = np.random.default_rng(0)
    planes = rng.integers(0, 2, (n, k // g, g, q)).astype(np.int8) * 2 - 1
    bw = o.to_kernel_layout(o.pack_binary_weight(planes))
    y = o.lutgemm_compute_shift_scale(np.zeros(n, np.float32), bw, alpha, x1)
    expect = 2.0 * 0.5 * planes.reshape(n, k, q)[:, 37, :].sum(axis=1)
    assert np.allclose(y, expect)


@pytest.fixture(scope="module")
def c_oracle():
    subprocess.run(["make", "-C", os.path.join(REPO, "oracle")], check=True, capture_output=True)
    return ctypes.CDLL(os.path.join(REPO, "oracle", "liblutgemv_oracle.so"))


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_c_restatement_matches_numpy(c_oracle):
    rng = np.random.default_rng(11)
    k, n, q, g, m = 128, 24, 3, 64, 2
    bw = rng.integers(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=np.int64).astype(np.int32)
    x = rng.standard_normal((m, k)).astype(np.float16)
    # mode A
    alpha = np.exp2(-rng.integers(2, 9, (k // g, q, n))).astype(np.float16)
    out = np.zeros(n, np.float32)
    assert c_oracle.ref_shift_scale(_ptr(out), _ptr(bw), _ptr(alpha), _ptr(x[0]), n, k, q, k // g) == 0
    assert o.max_rel_err(out, o.lutgemm_compute_shift_scale(np.zeros(n), bw, alpha, x[0])) < 1e-6
    # halving alpha + q_bias
    a1 = rng.random((k // g, n)).astype(np.float16)
    qb = (0.1 * rng.standard_normal((k // g, n))).astype(np.float16)
    out = np.zeros(n, np.float32)
    assert c_oracle.ref_compute(_ptr(out), _ptr(bw), _ptr(a1), _ptr(qb), _ptr(x[0]), n, k, q, k // g) == 0
    assert o.max_rel_err(out, o.lutgemm_compute(np.zeros(n), bw, a1, qb, x[0])) < 1e-6
    # block kernels
    ng = 3
    ab = rng.random((k // 8, q, ng)).astype(np.float16)
    out = np.zeros((m, n), np.float32)
    assert c_oracle.ref_block(_ptr(out), _ptr(bw), _ptr(ab), _ptr(x), m, n, k, q, ng) == 0
    assert o.max_rel_err(out, o.lutgemm_compute_block(np.zeros((m, n)), bw, ab, x)) < 1e-6
    au = rng.integers(0, 512, (k // 8, q, ng)).astype(np.uint16)
    out = np.zeros((m, n), np.float32)
    assert c_oracle.ref_block_shift(_ptr(out), _ptr(bw), _ptr(au), _ptr(x), m, n, k, q, ng) == 0
    assert o.max_rel_err(out, o.lutgemm_compute_block_shift(np.zeros((m, n)), bw, au, x)) < 1e-6
    ai = rng.integers(-9, -1, (k // 8, q, ng, 3)).astype(np.int8)
    ai[0, 0, 0, 1:] = o.APOT_NONE
    out = np.zeros((m, n), np.float32)
    assert c_oracle.ref_block_shift_int8(_ptr(out), _ptr(bw), _ptr(ai), _ptr(x), m, n, k, q, ng) == 0
    assert o.max_rel_err(out, o.lutgemm_compute_block_shift_int8(np.zeros((m, n)), bw, ai, x)) < 1e-6

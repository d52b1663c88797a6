"""CPU oracle for the BCQ LUT-GEMV path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy, the algorithm of the ShiftAddLLM reference for
its binary-coding-quantised (BCQ) weight x fp16 activation product.  It is the
checker the CUDA path is compared against: only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it.  The product package
never does; without its CUDA library the product raises.

Parity status: PINNED.  Every function here is checked against outputs of the
reference's own Python (imported unchanged, on CPU) stored under
``tests/golden`` by ``tests/golden/make_golden.py``.  The reference ships no
golden vectors of its own; its only self-check is the identity
``unpack_weight(pack_binaryWeight(B), alpha) == einsum(B, alpha)``
(zeroShot/models/kernel.py:96-120, quant_methods/shiftaddllm.py:204-207), which
is reproduced in the tests as well.

Naming: K = in_features, N = out_features, q = number of bit planes,
g = group size along K (mode A), gs = group size along N (mode B).
Kernel layout of the packed planes is uint32 ``[K/32][q][N]``: bit t of word kk
of column n is input feature 32*kk+t, set means +1
(lut_gemm/mv_fp16_bias.hpp:52,86-90 together with lut_gemm/kernel.py:19-21).
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------
# Packing (integer work, bit-exact)
# ----------------------------------------------------------------------------


def pack_binary_weight(b_weight: np.ndarray) -> np.ndarray:
    """+-1 planes ``[R, n_groups, group_size, q]`` -> int32 ``[R, C/32, q]``.

    Follows lut_gemm/kernel.py:9-23 (``pack_binaryWeight``): dims 1 and 2 are
    flattened to C, 32 consecutive elements along C go into one word, element
    32*j+t lands in bit t, a set bit means +1.  The reference sums
    ``bit * 2**t`` in int64 and narrows to int32, i.e. bit 31 wraps negative.
    """
    b = np.asarray(b_weight)
    if b.ndim != 4:
        raise ValueError(f"expected [R, n_groups, group_size, q], got {b.shape}")
    if not np.all((b == 1) | (b == -1)):
        raise ValueError("binary weight must hold only +1 / -1")
    r, ng, gsz, q = b.shape
    c = ng * gsz
    if c % 32:
        raise ValueError("packed dimension must be a multiple of 32")
    bits = (b.reshape(r, c // 32, 32, q) == 1).astype(np.uint64)
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64)).reshape(1, 1, 32, 1)
    words = (bits * weights).sum(axis=2)  # [R, C/32, q] uint64 < 2**32
    return words.astype(np.uint32).view(np.int32).copy()


def expand_bits(words: np.ndarray) -> np.ndarray:
    """int32/uint32 ``[..., W]`` -> uint8 ``[..., W, 32]``, entry t = bit t."""
    u = np.ascontiguousarray(words).view(np.uint32)
    shifts = np.arange(32, dtype=np.uint32)
    return ((u[..., None] >> shifts) & np.uint32(1)).astype(np.uint8)


def unpack_weight(bw: np.ndarray, alpha: np.ndarray) -> np.ndarray:
    """Dequantise: packed ``[R, C/32, q]`` + alpha ``[R, G, q]`` -> fp32 ``[R, C]``.

    Follows lut_gemm/kernel.py:26-56 (``unpack_weight``):
    ``W[r, c] = sum_b alpha[r, c // (C/G), b] * (2*bit_b(r, c) - 1)``.
    The reference starts from zero and adds plane b = 0, 1, ... in that order
    in fp32; the same order is kept so the result is bit-identical.
    """
    bw = np.asarray(bw)
    alpha = np.asarray(alpha, dtype=np.float32)
    r, w, q = bw.shape
    c = w * 32
    g = alpha.shape[1]
    if alpha.shape[0] != r or alpha.shape[2] != q:
        raise ValueError("alpha must be [R, G, q] matching the packed tensor")
    if c % g:
        raise ValueError("C must be divisible by the number of groups")
    gsz = c // g
    out = np.zeros((r, c), dtype=np.float32)
    for b in range(q):
        sign = expand_bits(bw[:, :, b]).reshape(r, c).astype(np.float32) * 2.0 - 1.0
        a = np.repeat(alpha[:, :, b], gsz, axis=1)  # [R, C]
        out += a * sign
    return out


def unpack_to_fake_binary_weight(bw: np.ndarray, n_groups: int = 1) -> np.ndarray:
    """Inverse of :func:`pack_binary_weight`: int32 ``[R, C/32, q]`` -> +-1
    ``[R, n_groups, C/n_groups, q]`` (lut_gemm/kernel.py:58-75; the reference
    computes ``bit*2-1`` in uint8, so -1 shows up as 255 there; here int8)."""
    bw = np.asarray(bw)
    r, w, q = bw.shape
    c = w * 32
    planes = [expand_bits(bw[:, :, b]).reshape(r, c).astype(np.int8) * 2 - 1 for b in range(q)]
    full = np.stack(planes, axis=-1)
    return full.reshape(r, n_groups, c // n_groups, q)


def to_kernel_layout(packed_rows: np.ndarray) -> np.ndarray:
    """``[N, K/32, q]`` (rows = output features, packed along K) ->
    kernel layout ``[K/32, q, N]`` (lut_gemm/kernel.py:29, hpp:52)."""
    return np.ascontiguousarray(np.transpose(packed_rows, (1, 2, 0)))


def convert_weight(bw_lat: np.ndarray, alpha_lat: np.ndarray):
    """Lat.-checkpoint layout -> kernel layout, for ANY shape.

    Input ``bw_lat`` int32 ``[K_in, N_out/32, q]`` is packed along out_features
    (quant_methods/shiftaddllm.py:193-202); the kernel wants words packed along
    in_features: ``P[kk, b, n] = sum_t 2**t * [B_b[32*kk+t, n] == +1]``.
    ``alpha_lat`` ``[R, G, q]`` -> fp32 ``[R, q, G]``.
    Restates lut_gemm/kernel.py:112-133 (``convert_weight``); that function
    agrees with this one for square layers and raises for others.
    """
    bw_lat = np.asarray(bw_lat)
    k_in, w, q = bw_lat.shape
    n_out = w * 32
    if k_in % 32:
        raise ValueError("in_features must be a multiple of 32")
    out = np.empty((k_in // 32, q, n_out), dtype=np.uint32)
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64)).reshape(1, 32, 1)
    for b in range(q):
        bits = expand_bits(bw_lat[:, :, b]).reshape(k_in, n_out).astype(np.uint64)
        out[:, b, :] = (bits.reshape(k_in // 32, 32, n_out) * weights).sum(axis=1).astype(np.uint32)
    alpha = np.ascontiguousarray(np.transpose(np.asarray(alpha_lat, dtype=np.float32), (0, 2, 1)))
    return out.view(np.int32), alpha


def planes_from_kernel_layout(bw_kernel: np.ndarray) -> np.ndarray:
    """Kernel layout ``[K/32, q, N]`` -> +-1 fp32 ``[q, K, N]``."""
    bw_kernel = np.asarray(bw_kernel)
    kw, q, n = bw_kernel.shape
    bits = expand_bits(np.transpose(bw_kernel, (1, 2, 0)))  # [q, N, K/32, 32]
    sign = bits.reshape(q, n, kw * 32).astype(np.float32) * 2.0 - 1.0
    return np.ascontiguousarray(np.transpose(sign, (0, 2, 1)))


# ----------------------------------------------------------------------------
# APoT exponents (lut_gemm/quant.py:30-39 + quantizers/bcq_quant/bcq_shift.py:15-24)
# ----------------------------------------------------------------------------

APOT_NONE = -128  # explicit "no term" code understood by the int8 entry point


def _shift_of(x: np.ndarray) -> np.ndarray:
    """``round(log(|x|)/log(2))`` in fp32 with round-half-to-even, the value the
    reference computes with ``torch.log`` and ``Tensor.round``."""
    with np.errstate(divide="ignore", invalid="ignore"):
        return np.rint(np.log(np.abs(x).astype(np.float32)) / np.float32(np.log(2)))


def quantize_to_apot(alpha: np.ndarray, num_apot: int = 3, *, mark_missing: bool = False) -> np.ndarray:
    """alpha -> ``num_apot`` int8 exponents per value, last dim appended.

    Restates ``LutLinear.quantize_to_apot`` (lut_gemm/quant.py:30-39).  Term 0
    is ``round(log2|a|)``; terms 1.. are ``round(log2|a - running|)`` where
    ``running`` accumulates ``sign * 2**shift``.  Only shifts are stored, signs
    of the residual terms are lost, exactly as upstream.  When the residual is
    zero the reference computes ``log2(0) = -inf`` and narrows it to int8, which
    gives 0 on x86 (a spurious ``2**0`` term); ``mark_missing=True`` writes
    :data:`APOT_NONE` there instead, which is what the new int8 kernel treats
    as "no term".
    """
    a = np.asarray(alpha, dtype=np.float32)
    running = np.zeros_like(a)
    cols = []
    for _ in range(num_apot):
        resid = a - running
        shift = _shift_of(resid)
        finite = np.isfinite(shift)
        code = np.where(finite, shift, 0.0)
        stored = np.clip(code, -128, 127).astype(np.int8)
        if mark_missing:
            stored = np.where(finite, stored, np.int8(APOT_NONE)).astype(np.int8)
        cols.append(stored)
        with np.errstate(over="ignore", invalid="ignore"):
            running = running + np.where(finite, np.exp2(code).astype(np.float32) * np.sign(resid), 0.0).astype(np.float32)
    return np.stack(cols, axis=-1)


# ----------------------------------------------------------------------------
# Layer outputs (floating point; the CUDA path must match within 1e-2 of max|y|)
# ----------------------------------------------------------------------------


def dequant_mode_a(bw_kernel: np.ndarray, alpha: np.ndarray) -> np.ndarray:
    """Mode A weight ``W[N, K]`` fp32 from kernel-layout planes ``[K/32, q, N]``
    and alpha ``[K/g, q, N]`` — the same numbers ``unpack_weight`` returns for
    ``packed[N, K/32, q]``, ``alpha[N, K/g, q]`` (lut_gemm/kernel.py:26-56)."""
    packed_rows = np.ascontiguousarray(np.transpose(np.asarray(bw_kernel), (2, 0, 1)))
    alpha_rows = np.ascontiguousarray(np.transpose(np.asarray(alpha, dtype=np.float32), (2, 0, 1)))
    return unpack_weight(packed_rows, alpha_rows)


def dequant_mode_b(bw_kernel: np.ndarray, alpha_mult: np.ndarray) -> np.ndarray:
    """Mode B weight ``W[N, K]``: one multiplier per (8 inputs x gs outputs)
    block, ``alpha_mult`` fp32 ``[K/8, q, N/gs]`` (hpp:158-208)."""
    sign = planes_from_kernel_layout(bw_kernel)  # [q, K, N]
    q, k, n = sign.shape
    a = np.asarray(alpha_mult, dtype=np.float32)
    ngroups = a.shape[2]
    gs = n // ngroups
    full = np.repeat(np.repeat(a, 8, axis=0), gs, axis=2)  # [K, q, N]
    w = np.zeros((k, n), dtype=np.float32)
    for b in range(q):
        w += full[:, b, :] * sign[b]
    return np.ascontiguousarray(w.T)


def linear_fp32(x: np.ndarray, w: np.ndarray, bias=None) -> np.ndarray:
    """``y = x.float() @ W.T (+ bias)`` — the reference's dequantise-then-matmul
    path (lut_gemm/kernel.py:101-107 followed by ``F.linear``), in fp32."""
    y = np.asarray(x, dtype=np.float32) @ np.asarray(w, dtype=np.float32).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)
    return y


def lutgemm_compute_shift_scale(output, bw_kernel, alpha, x):
    """``lutgemm_compute_shift_scale`` (lutgemm_cuda.cpp:43-52, hpp:498-579):
    ``output[n] += sum_g sum_b alpha[g,b,n] * (B_b x)_g``; returns fp32."""
    w = dequant_mode_a(bw_kernel, alpha)
    return np.asarray(output, dtype=np.float32) + linear_fp32(np.asarray(x).reshape(1, -1), w)[0]


def lutgemm_compute(output, bw_kernel, alpha, q_bias, x):
    """``lutgemm_compute`` (lutgemm_cuda.cpp:88-98, hpp:8-103): one alpha per
    (group, column) halved for every plane (``reg_a /= 2`` before use, so plane
    b is scaled by alpha / 2**(b+1)), plus ``q_bias[g, n] * sum_{k in g} x_k``."""
    bw_kernel = np.asarray(bw_kernel)
    kw, q, n = bw_kernel.shape
    a = np.asarray(alpha, dtype=np.float32)  # [G, N]
    scales = np.stack([a / np.float32(2 ** (b + 1)) for b in range(q)], axis=1)  # [G, q, N]
    y = lutgemm_compute_shift_scale(output, bw_kernel, scales, x)
    g = a.shape[0]
    xs = np.asarray(x, dtype=np.float32).reshape(g, -1).sum(axis=1)  # [G]
    return y + (np.asarray(q_bias, dtype=np.float32) * xs[:, None]).sum(axis=0)


def lutgemm_compute_block(output, bw_kernel, alpha, x):
    """``lutgemm_compute_block`` (lutgemm_cuda.cpp:54-63, hpp:105-220):
    alpha fp16 ``[K/8, q, N/gs]``, x ``[M, K]``, output ``[M, N]`` in/out."""
    w = dequant_mode_b(bw_kernel, np.asarray(alpha, dtype=np.float32))
    xm = np.asarray(x, dtype=np.float32).reshape(-1, w.shape[1])
    return np.asarray(output, dtype=np.float32).reshape(xm.shape[0], -1) + linear_fp32(xm, w)


def apot_u16_multiplier(alpha_u16: np.ndarray) -> np.ndarray:
    """Multiplier of ``lutgemm_compute_block_shift`` (hpp:294-297): three 3-bit
    exponent fields, ``2**(a&7) + 2**((a>>3)&7) + 2**((a>>6)&7)``."""
    a = np.asarray(alpha_u16).astype(np.uint16).astype(np.int64)
    return (np.exp2(a & 7) + np.exp2((a >> 3) & 7) + np.exp2((a >> 6) & 7)).astype(np.float32)


def apot_i8_multiplier(alpha_i8: np.ndarray) -> np.ndarray:
    """Multiplier of ``lutgemm_compute_block_shiftInt8`` (hpp:335-340,473-482):
    each of the trailing-dim int8 shifts s contributes ``2**s`` (the reference
    adds ``s << 10`` to the fp16 bit pattern, which is a multiplication by 2**s
    for normal values); :data:`APOT_NONE` contributes nothing."""
    a = np.asarray(alpha_i8).astype(np.int64)
    term = np.where(a == APOT_NONE, 0.0, np.exp2(a.astype(np.float64)))
    return term.sum(axis=-1).astype(np.float32)


def lutgemm_compute_block_shift(output, bw_kernel, alpha_u16, x):
    """``lutgemm_compute_block_shift`` (lutgemm_cuda.cpp:65-74, hpp:223-328)."""
    return lutgemm_compute_block(output, bw_kernel, apot_u16_multiplier(alpha_u16), x)


def lutgemm_compute_block_shift_int8(output, bw_kernel, alpha_i8, x):
    """``lutgemm_compute_block_shiftInt8`` (lutgemm_cuda.cpp:76-85, hpp:342-495)."""
    return lutgemm_compute_block(output, bw_kernel, apot_i8_multiplier(alpha_i8), x)


# ----------------------------------------------------------------------------
# LUT formulation (the arithmetic the kernels actually perform), small cases
# ----------------------------------------------------------------------------


def build_lut(x8: np.ndarray) -> np.ndarray:
    """256-entry table for one 8-activation chunk: entry i is
    ``sum_j (+x[j] if bit j of i else -x[j])`` (hpp:19-45)."""
    x8 = np.asarray(x8, dtype=np.float32)
    idx = np.arange(256, dtype=np.uint32)
    sign = ((idx[:, None] >> np.arange(8, dtype=np.uint32)) & 1).astype(np.float32) * 2.0 - 1.0
    return sign @ x8


def lut_gemv_mode_a(bw_kernel, alpha, x) -> np.ndarray:
    """Mode A product by table gathers, pure loops over words: byte j of word
    kk indexes the table of chunk 4*kk+j (hpp:86-90, 551-566).  Slow; use on
    small shapes to pin the bit/byte conventions against :func:`dequant_mode_a`."""
    bw = np.ascontiguousarray(bw_kernel).view(np.uint32)
    kw, q, n = bw.shape
    a = np.asarray(alpha, dtype=np.float32)
    g = (kw * 32) // a.shape[0]
    xs = np.asarray(x, dtype=np.float32).reshape(-1)
    luts = np.stack([build_lut(xs[8 * c: 8 * c + 8]) for c in range(kw * 4)])  # [K/8, 256]
    y = np.zeros(n, dtype=np.float64)
    for kk in range(kw):
        grp = (kk * 32) // g
        for b in range(q):
            word = bw[kk, b]
            part = np.zeros(n, dtype=np.float64)
            for j in range(4):
                part += luts[4 * kk + j][(word >> np.uint32(8 * j)) & np.uint32(255)]
            y += a[grp, b].astype(np.float64) * part
    return y.astype(np.float32)


def max_rel_err(y, y_ref) -> float:
    """The acceptance metric: ``max|y - y_ref| / max|y_ref|``."""
    y = np.asarray(y, dtype=np.float64)
    r = np.asarray(y_ref, dtype=np.float64)
    denom = np.max(np.abs(r))
    return float(np.max(np.abs(y - r)) / (denom if denom > 0 else 1.0))

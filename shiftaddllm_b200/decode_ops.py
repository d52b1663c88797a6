"""Python face of include/sal_decode_ops.h: the fused steps between the LUT-GEMV calls of a
batch-1 decode step.  Tensors must be contiguous CUDA tensors; launches go to torch's current
stream and are CUDA-graph capturable (the position is read from a device tensor)."""
from __future__ import annotations

import torch

from . import _lib


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def residual_rmsnorm(x, delta, weight, out, x_out, eps: float):
    """t = x (+ delta); x_out = t (if given, may be x itself); out = rmsnorm(t) * weight."""
    lib = _lib.load()
    _lib.check(lib.sal_residual_rmsnorm_f16(x.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
                                            out.data_ptr(), None if x_out is None else x_out.data_ptr(), x.numel(),
                                            float(eps), _stream(x)), "sal_residual_rmsnorm_f16")


def rope_kv_write(q, k, v, cos, sin, pos, k_cache, v_cache, heads, kv_heads, hd):
    lib = _lib.load()
    _lib.check(lib.sal_rope_kv_write_f16(q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                         pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), heads, kv_heads, hd,
                                         k_cache.shape[0], _stream(q)), "sal_rope_kv_write_f16")


def residual_rmsnorm_fixedacc(x, delta32, weight, out, x_out, eps: float, zero_a=None, zero_b=None):
    """As residual_rmsnorm with an int64 fixed-point accumulator as delta (consumed and zeroed); zero_a / zero_b:
    further accumulators to clear."""
    lib = _lib.load()
    _lib.check(lib.sal_residual_rmsnorm_fixedacc(x.data_ptr(), None if delta32 is None else delta32.data_ptr(), weight.data_ptr(),
                                               out.data_ptr(), None if x_out is None else x_out.data_ptr(), x.numel(), float(eps),
                                               None if zero_a is None else zero_a.data_ptr(), 0 if zero_a is None else zero_a.numel(),
                                               None if zero_b is None else zero_b.data_ptr(), 0 if zero_b is None else zero_b.numel(),
                                               _stream(x)), "sal_residual_rmsnorm_fixedacc")


def rope_kv_write_fixedacc(q32, k32, v32, q_out, cos, sin, pos, k_cache, v_cache, heads, kv_heads, hd):
    lib = _lib.load()
    _lib.check(lib.sal_rope_kv_write_fixedacc(q32.data_ptr(), k32.data_ptr(), v32.data_ptr(), q_out.data_ptr(), cos.data_ptr(),
                                            sin.data_ptr(), pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), heads,
                                            kv_heads, hd, k_cache.shape[0], _stream(q_out)), "sal_rope_kv_write_fixedacc")


def attention_workspace(heads: int, hd: int, device) -> torch.Tensor:
    """Zero-filled scratch for the split form of attention_decode (one per stream that uses it)."""
    lib = _lib.load()
    return torch.zeros(lib.sal_attention_workspace_bytes(int(heads), int(hd)), dtype=torch.uint8, device=device)


def attention_decode(q, k_cache, v_cache, pos, out, heads, kv_heads, hd, scale: float, workspace=None):
    """Single-query attention over cache positions 0..pos.  With a `workspace` (attention_workspace) the
    positions are split over many CTAs and merged; shapes that form does not take fall back to one CTA
    per head."""
    lib = _lib.load()
    if workspace is not None:
        rc = lib.sal_attention_decode_split_f16(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(),
                                                out.data_ptr(), heads, kv_heads, hd, k_cache.shape[0], float(scale),
                                                workspace.data_ptr(), workspace.numel(), _stream(q))
        if rc != _lib.SAL_E_UNSUPPORTED:
            _lib.check(rc, "sal_attention_decode_split_f16")
            return
    _lib.check(lib.sal_attention_decode_f16(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(),
                                            out.data_ptr(), heads, kv_heads, hd, k_cache.shape[0], float(scale),
                                            _stream(q)), "sal_attention_decode_f16")


def rope_attention_decode(q, k_new, v_new, cos, sin, pos, k_cache, v_cache, out, heads, kv_heads, hd, scale: float, workspace):
    """Rotary step of the new token, cache write and split attention in one kernel.  q / k_new / v_new: fp16
    projections (left untouched) or int64 fixed-point accumulators (consumed and cleared).  Returns False — having done
    nothing — for shapes the split kernel does not take."""
    lib = _lib.load()
    f32 = q.dtype == torch.int64          # fixed-point accumulators (consumed and cleared)
    if k_new.dtype != q.dtype or v_new.dtype != q.dtype or q.dtype not in (torch.float16, torch.int64):
        raise RuntimeError("q, k_new and v_new must all be float16 or all int64 fixed-point accumulators")
    rc = lib.sal_rope_attention_decode(q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), 1 if f32 else 0, cos.data_ptr(),
                                       sin.data_ptr(), pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                       heads, kv_heads, hd, k_cache.shape[0], float(scale), workspace.data_ptr(),
                                       workspace.numel(), _stream(out))
    if rc == _lib.SAL_E_UNSUPPORTED:
        return False
    _lib.check(rc, "sal_rope_attention_decode")
    return True


def residual_rmsnorm_rows(x, delta, weight, out, x_out, eps: float):
    """residual_rmsnorm for every row of [rows, n] tensors (one weight vector)."""
    lib = _lib.load()
    rows, n = x.shape[0], x.shape[1]
    _lib.check(lib.sal_residual_rmsnorm_rows_f16(x.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
                                                 out.data_ptr(), None if x_out is None else x_out.data_ptr(), rows, n, float(eps),
                                                 _stream(x)), "sal_residual_rmsnorm_rows_f16")


def attention_workspace_batch(batch: int, heads: int, hd: int, device) -> torch.Tensor:
    lib = _lib.load()
    return torch.zeros(int(batch) * lib.sal_attention_workspace_bytes(int(heads), int(hd)), dtype=torch.uint8, device=device)


def rope_attention_decode_batch(q, k_new, v_new, cos, sin, pos, k_cache, v_cache, out, heads, kv_heads, hd, scale: float, workspace):
    """rope_attention_decode for `batch` sequences in lock step: q [batch, heads*hd], k_new / v_new [batch, kv_heads*hd] (fp16),
    caches [batch, max_len, kv_heads, hd], out [batch, heads*hd].  Returns False — having done nothing — for shapes
    the split kernel does not take."""
    lib = _lib.load()
    rc = lib.sal_rope_attention_decode_batch(q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                             pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), q.shape[0], heads,
                                             kv_heads, hd, k_cache.shape[1], float(scale), workspace.data_ptr(), workspace.numel(),
                                             _stream(out))
    if rc == _lib.SAL_E_UNSUPPORTED:
        return False
    _lib.check(rc, "sal_rope_attention_decode_batch")
    return True


def greedy_token(logits_f16, logits_f32, token, pos):
    """End of a greedy step in one launch: fp32 copy of the fp16 logits (``logits_f32`` may be None), ``token[0]`` =
    argmax (first of equal maxima), ``pos[0] += 1``.  False if the vocabulary size is not a multiple of 8."""
    vocab = logits_f16.numel()
    if vocab % 8 != 0 or logits_f16.dtype != torch.float16 or not logits_f16.is_contiguous():
        return False
    lib = _lib.load()
    _lib.check(lib.sal_greedy_token_f16(logits_f16.data_ptr(), logits_f32.data_ptr() if logits_f32 is not None else None, vocab,
                                        token.data_ptr(), pos.data_ptr(), _stream(logits_f16)), "sal_greedy_token_f16")
    return True


def silu_mul(gate, up, out):
    lib = _lib.load()
    _lib.check(lib.sal_silu_mul_f16(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _stream(gate)),
               "sal_silu_mul_f16")

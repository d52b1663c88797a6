"""ctypes binding of ``libsal_lutgemm.so`` (the C ABI in ``include/sal_lutgemm.h``).

There is no CPU fallback: if the shared library is missing the import of any
compute function raises, and on a machine without a compute-capability 10.x
GPU every compute call returns ``SAL_E_DEVICE`` which is raised as
``RuntimeError``.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# SAL_LUTGEMM_LIBRARY names another build of the same library (e.g. one compiled with -DSAL_MEASURE)
LIB_PATH = os.environ.get("SAL_LUTGEMM_LIBRARY") or os.path.join(_PKG_DIR, "libsal_lutgemm.so")

SAL_OK = 0
SAL_E_NULL, SAL_E_SHAPE, SAL_E_ALIGN, SAL_E_WORKSPACE = -1, -2, -3, -4
SAL_E_LAUNCH, SAL_E_UNSUPPORTED, SAL_E_DEVICE, SAL_E_TIMEOUT = -5, -6, -7, -8
SAL_ACCUMULATE, SAL_PDL, SAL_FORCE_GENERIC, SAL_OUT_FIXED_ATOMIC, SAL_SWIGLU_FIXED = 1, 2, 4, 8, 16
SAL_MAX_GROUP = 8
SAL_MAX_PEERS = 8
SAL_MAX_M = 64

_vp, _i, _u, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t


class SalProblem(ctypes.Structure):
    _fields_ = [("bw", _vp), ("alpha", _vp), ("bias", _vp), ("x", _vp), ("y", _vp),
                ("M", _i), ("K", _i), ("N", _i), ("q", _i), ("num_groups", _i), ("x_mul", _vp)]


class SalExchange(ctypes.Structure):
    _fields_ = [("world", _i), ("rank", _i), ("slot", _i), ("peer_buffers", _vp * 8), ("peer_flags", _vp * 8),
                ("gather_offsets", ctypes.POINTER(ctypes.c_longlong))]


class SalPlanInfo(ctypes.Structure):
    _fields_ = [("tiled", _i), ("ctas", _i), ("ranges", _i), ("splits", _i), ("stages", _i), ("smem_bytes", _i)]


# name -> (restype, argtypes); mirrors include/sal_lutgemm.h one to one
SIGNATURES = {
    "sal_version": (_i, []),
    "sal_status_string": (ctypes.c_char_p, [_i]),
    "sal_last_cuda_error": (ctypes.c_char_p, []),
    "sal_device_ok": (_i, []),
    "sal_workspace_bytes": (_sz, [_i, _i]),
    "sal_workspace_status": (_i, [_vp, _vp]),
    "sal_lutgemv_shift_scale": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _u, _vp, _sz, _vp]),
    "sal_lutgemv_shift_scale_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _u, _vp]),
    "sal_static_status": (_i, [_vp]),
    "sal_lutgemv_compute": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _u, _vp, _sz, _vp]),
    "sal_lutgemm_block": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _u, _vp, _sz, _vp]),
    "sal_lutgemm_block_shift": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _u, _vp, _sz, _vp]),
    "sal_lutgemm_block_shift_int8": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _u, _vp, _sz, _vp]),
    "sal_lutgemv_grouped": (_i, [ctypes.POINTER(SalProblem), _i, _u, _vp, _sz, _vp]),
    "sal_lutgemv_grouped_exchange": (_i, [ctypes.POINTER(SalProblem), _i, _u, _vp, _sz, ctypes.POINTER(SalExchange),
                                          ctypes.POINTER(_i), _vp]),
    "sal_exchange_wait": (_i, [_vp, _i, _u, _vp, _vp]),
    "sal_prepare_grouped": (_i, [ctypes.POINTER(SalProblem), _i, _u, ctypes.POINTER(SalExchange), ctypes.POINTER(_vp)]),
    "sal_prepared_workspace_bytes": (_sz, [_vp]),
    "sal_prepared_writers": (_i, [_vp]),
    "sal_launch_prepared": (_i, [_vp, _vp, _sz, _i, _vp]),
    "sal_launch_prepared_sequence": (_i, [ctypes.POINTER(_vp), _i, ctypes.POINTER(_i), _vp, _sz, _vp]),
    "sal_destroy_prepared": (None, [_vp]),
    "sal_plan_shift_scale": (_i, [_i, _i, _i, _i, _i, ctypes.POINTER(SalPlanInfo)]),
    # include/sal_decode_ops.h
    "sal_residual_rmsnorm_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, ctypes.c_float, _vp]),
    "sal_rope_kv_write_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "sal_residual_rmsnorm_fixedacc": (_i, [_vp, _vp, _vp, _vp, _vp, _i, ctypes.c_float, _vp, _i, _vp, _i, _vp]),
    "sal_rope_kv_write_fixedacc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "sal_attention_decode_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, ctypes.c_float, _vp]),
    "sal_attention_workspace_bytes": (ctypes.c_size_t, [_i, _i]),
    "sal_attention_decode_split_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, ctypes.c_float, _vp, ctypes.c_size_t, _vp]),
    "sal_pack_planes_i8": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "sal_repack_lat_to_kernel": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "sal_rope_attention_decode": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, ctypes.c_float, _vp,
                                       ctypes.c_size_t, _vp]),
    "sal_silu_mul_f16": (_i, [_vp, _vp, _vp, _i, _vp]),
    "sal_greedy_token_f16": (_i, [_vp, _vp, _i, _vp, _vp, _vp]),
    "sal_residual_rmsnorm_rows_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, ctypes.c_float, _vp]),
    "sal_rope_attention_decode_batch": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, ctypes.c_float, _vp,
                                            ctypes.c_size_t, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m shiftaddllm_b200.build` "
                "(there is no CPU or PyTorch fallback for the LUT-GEMV path)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        if hasattr(lib, "sal_debug_set"):   # present only in measurement builds (-DSAL_MEASURE)
            lib.sal_debug_set.restype = _i
            lib.sal_debug_set.argtypes = [ctypes.c_char_p, _i]
            lib.sal_debug_read.restype = _i
            lib.sal_debug_read.argtypes = [_vp, _sz]
        _lib = lib
    return _lib


def status_string(code: int) -> str:
    return load().sal_status_string(code).decode()


def check(code: int, what: str) -> None:
    if code != SAL_OK:
        detail = f"; CUDA: {load().sal_last_cuda_error().decode()}" if code == SAL_E_LAUNCH else ""
        raise RuntimeError(f"{what} failed: {status_string(code)} (status {code}){detail}")

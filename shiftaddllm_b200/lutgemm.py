"""Drop-in for the reference's compiled ``lutgemm`` extension.

Same five function names, argument order and in-place accumulate semantics as
lut_gemm/lutgemm_cuda.cpp:43-98, 225-230; the work is done by the sm_100a
library behind the C ABI of ``include/sal_lutgemm.h``.  To make reference code
that does ``import lutgemm`` pick this module up, call :func:`install`.

Differences from the reference, all deliberate: arguments are validated
(dtype, device, contiguity, shapes) and a bad call raises ``RuntimeError``
instead of reading out of bounds; kernels run on torch's current stream, not
the legacy default stream; accumulation is fp32 and deterministic; batch
(``M > 1``) inputs are accepted by every entry point.
"""
from __future__ import annotations

import ctypes
import os
import sys

import torch

from . import _lib

FIXED_ONE = float(2 ** 32)   # value of 1.0 in a fixed-point accumulator (SAL_OUT_FIXED_ATOMIC)

_workspaces: dict = {}
_superseded: list = []   # outgrown scratch buffers: kept alive, a CUDA graph captured earlier may still name them


def workspace_bytes(device: torch.device, need: int) -> torch.Tensor:
    """Zero-initialised scratch for the split-K reduction, cached per
    (device, stream) and grown on demand.  Calls on one stream are ordered, so
    sharing one buffer per stream is race-free.  A buffer that is outgrown is
    kept (not freed): launches captured into a CUDA graph keep using the address
    they were captured with, and the old buffer stays valid for them."""
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _superseded.append(ws)
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def workspace_for(device: torch.device, m: int, n: int) -> torch.Tensor:
    """Scratch large enough for a product (or a group of products) with `m` rows and `n` columns in all."""
    return workspace_bytes(device, _lib.load().sal_workspace_bytes(m, n))


def _req(t: torch.Tensor, dtype, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _rows(output: torch.Tensor, d_input: torch.Tensor, n: int, k: int):
    if d_input.numel() % k or output.numel() % n:
        raise RuntimeError("input/output sizes do not match kSize/mSize")
    m = d_input.numel() // k
    if output.numel() // n != m:
        raise RuntimeError(f"output holds {output.numel() // n} rows but input holds {m}")
    return m


def _launch(fn_name, output, bWeight, alpha, alpha_dtype, d_input, mSize, kSize, nb, num_groups, *,
            extra_ptr=None, num_apot=None, alpha_numel=None, flags=_lib.SAL_ACCUMULATE, bias=None):
    lib = _lib.load()
    _req(output, torch.float16, "output")
    _req(bWeight, torch.int32, "bWeight")
    _req(alpha, alpha_dtype, "alpha")
    _req(d_input, torch.float16, "d_input")
    n, k, q = int(mSize), int(kSize), int(nb)
    if k % 32 or bWeight.numel() != (k // 32) * q * n:
        raise RuntimeError(f"bWeight must hold (kSize/32)*nb*mSize = {(k // 32) * q * n} words, has {bWeight.numel()}")
    if alpha_numel is not None and alpha.numel() != alpha_numel:
        raise RuntimeError(f"alpha must hold {alpha_numel} elements, has {alpha.numel()}")
    m = _rows(output, d_input, n, k)
    dev = output.device
    for t in (bWeight, alpha, d_input):
        if t.device != dev:
            raise RuntimeError("all tensors must live on the same device")
    with torch.cuda.device(dev):
        ws = workspace_for(dev, m, n)
        stream = torch.cuda.current_stream(dev).cuda_stream
        args = [bWeight.data_ptr(), alpha.data_ptr()]
        if extra_ptr is not None:
            args.append(extra_ptr)
        args += [bias.data_ptr() if bias is not None else None, d_input.data_ptr(), output.data_ptr(), m, k, n, q,
                 int(num_groups)]
        if num_apot is not None:
            args.append(int(num_apot))
        args += [flags, ws.data_ptr(), ws.numel(), stream]
        _lib.check(getattr(lib, fn_name)(*args), fn_name)


def lutgemm_compute_shift_scale(output, bWeight, alpha, d_input, mSize, kSize, nb, num_groups):
    """``output += sum_b alpha[g,b,:] * (B_b^T x)``; alpha fp16 ``[num_groups, nb, mSize]``
    (lutgemm_cuda.cpp:43-52)."""
    _launch("sal_lutgemv_shift_scale", output, bWeight, alpha, torch.float16, d_input, mSize, kSize, nb, num_groups,
            alpha_numel=int(num_groups) * int(nb) * int(mSize))


def lutgemm_compute(output, bWeight, alpha, q_bias, d_input, mSize, kSize, nb, num_groups):
    """alpha, q_bias fp16 ``[num_groups, mSize]``; plane b scaled by ``alpha / 2**(b+1)``
    (lutgemm_cuda.cpp:88-98)."""
    _req(q_bias, torch.float16, "q_bias")
    if q_bias.numel() != int(num_groups) * int(mSize):
        raise RuntimeError("q_bias must hold num_groups*mSize elements")
    _launch("sal_lutgemv_compute", output, bWeight, alpha, torch.float16, d_input, mSize, kSize, nb, num_groups,
            extra_ptr=q_bias.data_ptr(), alpha_numel=int(num_groups) * int(mSize))


def lutgemm_compute_block(output, bWeight, alpha, d_input, mSize, kSize, nb, num_groups):
    """alpha fp16 ``[kSize/8, nb, num_groups]`` (lutgemm_cuda.cpp:54-63)."""
    _launch("sal_lutgemm_block", output, bWeight, alpha, torch.float16, d_input, mSize, kSize, nb, num_groups,
            alpha_numel=(int(kSize) // 8) * int(nb) * int(num_groups))


def lutgemm_compute_block_shift(output, bWeight, alpha, d_input, mSize, kSize, nb, num_groups, num_apot):
    """alpha int16 ``[kSize/8, nb, num_groups]``, three 3-bit exponents (lutgemm_cuda.cpp:65-74)."""
    _launch("sal_lutgemm_block_shift", output, bWeight, alpha, torch.int16, d_input, mSize, kSize, nb, num_groups,
            alpha_numel=(int(kSize) // 8) * int(nb) * int(num_groups))


def lutgemm_compute_block_shiftInt8(output, bWeight, alpha, d_input, mSize, kSize, nb, num_groups, num_apot):
    """alpha int8 ``[kSize/8, nb, num_groups, num_apot]`` (lutgemm_cuda.cpp:76-85); -128 = no term."""
    _launch("sal_lutgemm_block_shift_int8", output, bWeight, alpha, torch.int8, d_input, mSize, kSize, nb, num_groups,
            num_apot=num_apot, alpha_numel=(int(kSize) // 8) * int(nb) * int(num_groups) * int(num_apot))


def lutgemv_fused(output, bWeight, alpha, bias, d_input, mSize, kSize, nb, num_groups, *, pdl=False):
    """Extension over the reference API: ``output = bias + product`` in one
    kernel (no separate ``bias.clone()``), optionally launched with programmatic
    dependent launch."""
    flags = _lib.SAL_PDL if pdl else 0
    _launch("sal_lutgemv_shift_scale", output, bWeight, alpha, torch.float16, d_input, mSize, kSize, nb, num_groups,
            flags=flags, bias=bias, alpha_numel=int(num_groups) * int(nb) * int(mSize))


def lutgemm_block_fused(output, bWeight, alpha, bias, d_input, mSize, kSize, nb, num_groups, *, pdl=False):
    """Extension over the reference API, block (mode B) layouts: ``output = bias + product`` in one
    kernel.  The multiplier encoding follows alpha's dtype: float16 ``[kSize/8, nb, num_groups]``,
    int16 (three 3-bit exponents) of the same shape, or int8 ``[kSize/8, nb, num_groups, num_apot]``."""
    flags = _lib.SAL_PDL if pdl else 0
    numel = (int(kSize) // 8) * int(nb) * int(num_groups)
    if alpha.dtype == torch.float16:
        _launch("sal_lutgemm_block", output, bWeight, alpha, torch.float16, d_input, mSize, kSize, nb, num_groups,
                flags=flags, bias=bias, alpha_numel=numel)
    elif alpha.dtype == torch.int16:
        _launch("sal_lutgemm_block_shift", output, bWeight, alpha, torch.int16, d_input, mSize, kSize, nb, num_groups,
                flags=flags, bias=bias, alpha_numel=numel)
    elif alpha.dtype == torch.int8:
        if alpha.dim() != 4:
            raise RuntimeError("int8 alpha must be [kSize/8, nb, num_groups, num_apot]")
        _launch("sal_lutgemm_block_shift_int8", output, bWeight, alpha, torch.int8, d_input, mSize, kSize, nb, num_groups,
                num_apot=alpha.shape[3], flags=flags, bias=bias, alpha_numel=numel * alpha.shape[3])
    else:
        raise RuntimeError(f"unsupported alpha dtype {alpha.dtype}")


def marshal_problems(problems, *, atomic_fixed=False, swiglu_fixed=False):
    """Checks the tensors of a grouped launch and returns (ctypes array, tensors to keep alive)."""
    if not 1 <= len(problems) <= _lib.SAL_MAX_GROUP:
        raise RuntimeError(f"a grouped launch takes 1..{_lib.SAL_MAX_GROUP} problems")
    arr = (_lib.SalProblem * len(problems))()
    keep = []
    out_dtype = torch.int64 if atomic_fixed else torch.float16     # fixed-point accumulators: int64, units of 2**-32
    in_dtype = torch.int64 if swiglu_fixed else torch.float16
    for i, p in enumerate(problems):
        _req(p["output"], out_dtype, "output")
        _req(p["bWeight"], torch.int32, "bWeight")
        _req(p["alpha"], torch.float16, "alpha")
        _req(p["d_input"], in_dtype, "d_input")
        n, k = int(p["mSize"]), int(p["kSize"])
        m = _rows(p["output"], p["d_input"], n, k)
        bias = p.get("bias")
        mul = p.get("d_input_mul")      # optional: the activation is silu(d_input) * d_input_mul
        if mul is not None:
            _req(mul, in_dtype, "d_input_mul")
            if mul.numel() != p["d_input"].numel():
                raise RuntimeError("d_input_mul must have the shape of d_input")
        arr[i] = _lib.SalProblem(p["bWeight"].data_ptr(), p["alpha"].data_ptr(),
                                 bias.data_ptr() if bias is not None else None, p["d_input"].data_ptr(),
                                 p["output"].data_ptr(), m, k, n, int(p["nb"]), int(p["num_groups"]),
                                 mul.data_ptr() if mul is not None else None)
        keep.append((p["output"], p["bWeight"], p["alpha"], bias, p["d_input"], mul))
    return arr, keep


class GroupedLaunch:
    """A grouped launch prepared once (``sal_prepare_grouped``: arguments validated, work split
    planned, tensor-map descriptors encoded); calling it enqueues the launch on the current stream
    of the tensors' device.  The tensors named at preparation are referenced, not copied: their
    storage must stay where it is.  Problems may differ in ``nb`` (mixed precision): the launch is
    then one kernel per distinct plane count."""

    def __init__(self, problems, *, pdl=False, accumulate=False, atomic_fixed=False, swiglu_fixed=False, exchange=None):
        self._lib = _lib.load()
        self._arr, self._keep = marshal_problems(problems, atomic_fixed=atomic_fixed, swiglu_fixed=swiglu_fixed)
        self._device = problems[0]["output"].device
        if self._device.index is None:
            self._device = torch.device("cuda", torch.cuda.current_device())
        self._flags = ((_lib.SAL_PDL if pdl else 0) | (_lib.SAL_ACCUMULATE if accumulate else 0)
                       | (_lib.SAL_OUT_FIXED_ATOMIC if atomic_fixed else 0) | (_lib.SAL_SWIGLU_FIXED if swiglu_fixed else 0))
        self._exchange = exchange          # a ctypes SalExchange (and what it points to), or None
        handle = _lib._vp()
        with torch.cuda.device(self._device):
            rc = self._lib.sal_prepare_grouped(self._arr, len(problems), self._flags,
                                               ctypes.byref(exchange[0]) if exchange is not None else None, ctypes.byref(handle))
        if rc != 0:
            _lib.check(rc, "sal_prepare_grouped")
        self._handle = handle
        self._need = self._lib.sal_prepared_workspace_bytes(handle)
        self.writers = self._lib.sal_prepared_writers(handle)
        self._launch = self._lib.sal_launch_prepared

    def __call__(self, slot: int = -1):
        dev = self._device
        if torch.cuda.current_device() != dev.index:
            with torch.cuda.device(dev):
                return self(slot)
        stream = torch.cuda.current_stream(dev).cuda_stream
        ws = _workspaces.get((dev.index, stream))
        if ws is None or ws.numel() < self._need:
            ws = workspace_bytes(dev, self._need)
        rc = self._launch(self._handle, ws.data_ptr(), ws.numel(), slot, stream)
        if rc != 0:
            _lib.check(rc, "sal_launch_prepared")

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.sal_destroy_prepared(handle)


class LaunchSequence:
    """Several prepared launches enqueued by one call into the library (`sal_launch_prepared_sequence`): what a
    decoder block or a whole token is.  All launches must belong to one device."""

    def __init__(self, launches):
        self._launches = list(launches)
        if not self._launches:
            raise RuntimeError("an empty launch sequence")
        self._lib = _lib.load()
        self._device = self._launches[0]._device
        if any(l._device != self._device for l in self._launches):
            raise RuntimeError("all launches of a sequence must be on one device")
        self._handles = (_lib._vp * len(self._launches))(*[l._handle for l in self._launches])
        self._need = max(l._need for l in self._launches)

    def __call__(self):
        dev = self._device
        if torch.cuda.current_device() != dev.index:
            with torch.cuda.device(dev):
                return self()
        stream = torch.cuda.current_stream(dev).cuda_stream
        ws = _workspaces.get((dev.index, stream))
        if ws is None or ws.numel() < self._need:
            ws = workspace_bytes(dev, self._need)
        rc = self._lib.sal_launch_prepared_sequence(self._handles, len(self._launches), None, ws.data_ptr(), ws.numel(), stream)
        if rc != 0:
            _lib.check(rc, "sal_launch_prepared_sequence")


def prepare_grouped(problems, **kwargs) -> GroupedLaunch:
    """``lutgemv_grouped`` split in two: the checks and the marshalling happen here, once; the returned
    object is called every time the launch is wanted (a few microseconds of host time per call)."""
    return GroupedLaunch(problems, **kwargs)


def lutgemv_grouped(problems, *, pdl=False, accumulate=False, atomic_fixed=False, swiglu_fixed=False):
    """Several independent mode-A products in one launch.  ``problems`` is a list
    of dicts with keys output, bWeight, alpha, bias (or None), d_input,
    mSize, kSize, nb, num_groups and optionally d_input_mul (the activation is then
    silu(d_input) * d_input_mul, computed while the tables are built).

    ``atomic_fixed=True``: every ``output`` is an int64 fixed-point accumulator (units of 2**-32, see
    :data:`FIXED_ONE`) the product is ADDED to with integer atomics: no split-K reduction tail, and — integer
    sums being independent of the order of arrival — still bit-identical from run to run.
    ``swiglu_fixed=True``: d_input and d_input_mul are such accumulators."""
    GroupedLaunch(problems, pdl=pdl, accumulate=accumulate, atomic_fixed=atomic_fixed, swiglu_fixed=swiglu_fixed)()


def compiled_module():
    """The compiled `lutgemm` extension module (pybind11 + torch tensors over the C ABI; built by
    ``python -m shiftaddllm_b200.build`` into ``shiftaddllm_b200/ext/``), imported from there."""
    import importlib.util

    from . import build

    path = build.extension_path()
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `python -m shiftaddllm_b200.build`")
    spec = importlib.util.spec_from_file_location("lutgemm", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def install(name: str = "lutgemm", compiled: bool = True):
    """Makes ``import lutgemm`` (lut_gemm/quant.py:5) bind to this build, so that unmodified reference
    code runs on the sm_100a library.  ``compiled=True`` registers the compiled extension module — what
    lut_gemm/setup_lut.py installs for the reference; ``compiled=False`` registers this Python module
    (same five functions through ctypes).  Returns the registered module."""
    module = compiled_module() if compiled else sys.modules[__name__]
    sys.modules[name] = module
    return module

"""Packing, unpacking and checkpoint loading for BCQ weights (host side).

Mirrors the interface of the reference's ``lut_gemm/kernel.py`` — same function
names, argument meaning and tensor layouts — with vectorised torch code that
runs on whatever device its inputs live on.  Integer results are bit-exact
with the reference functions (see tests/test_host_logic.py for the CPU code and
tests/test_gpu_packing.py for the CUDA packers).
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn

from .quant import LutLinear, make_lut

__all__ = [
    "pack_binaryWeight", "pack_to_kernel_layout", "unpack_weight", "unpack_to_fake_binaryWeight", "convert_weight", "to_kernel_layout",
    "find_layers", "load_shiftaddllm_weight", "load_shiftaddllm_weight_with_kernel", "save_lat_checkpoint",
]


def _bit_weights(device) -> torch.Tensor:
    return torch.ones(32, dtype=torch.int64, device=device) << torch.arange(32, dtype=torch.int64, device=device)


def _pack_along(bits_le: torch.Tensor, dim: int) -> torch.Tensor:
    """Packs a {0,1} tensor along ``dim`` (length multiple of 32), element 32*j+t
    into bit t of word j; returns int32 with the packed dim in place."""
    moved = bits_le.movedim(dim, -1)
    shape = moved.shape[:-1] + (moved.shape[-1] // 32, 32)
    words = (moved.reshape(shape).to(torch.int64) * _bit_weights(bits_le.device)).sum(-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    return words.movedim(-1, dim)


def _unpack_along(words: torch.Tensor, dim: int) -> torch.Tensor:
    """Inverse of :func:`_pack_along`: int32 -> bool, ``dim`` grows 32x."""
    moved = words.movedim(dim, -1).to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(32, dtype=torch.int64, device=words.device)
    bits = ((moved.unsqueeze(-1) >> shifts) & 1).bool()
    return bits.flatten(-2).movedim(-1, dim)


def _pack_planes_cuda(bWeight: torch.Tensor, kernel_layout: bool) -> torch.Tensor:
    """CUDA tensors: one pass of ``sal_pack_planes_i8`` over the +-1 planes (the step the reference
    leaves on the CPU, model/opt.py:287)."""
    from . import _lib

    lib = _lib.load()
    r, ng, gsz, q = bWeight.shape
    c = ng * gsz
    signs = bWeight.to(torch.int8).contiguous()
    out = torch.empty((c // 32, q, r) if kernel_layout else (r, c // 32, q), dtype=torch.int32, device=bWeight.device)
    bad = torch.zeros(1, dtype=torch.int32, device=bWeight.device)
    with torch.cuda.device(bWeight.device):
        _lib.check(lib.sal_pack_planes_i8(signs.data_ptr(), out.data_ptr(), r, c, q, 1 if kernel_layout else 0, bad.data_ptr(),
                                          torch.cuda.current_stream(bWeight.device).cuda_stream), "sal_pack_planes_i8")
    if int(bad.item()):
        raise ValueError("BinaryWeight should be 1 or -1, but got other values")
    return out


def pack_to_kernel_layout(bWeight: torch.Tensor) -> torch.Tensor:
    """``[N, n_groups, group_size, wbit]`` of +-1 -> int32 ``[K/32, wbit, N]``: ``pack_binaryWeight``
    followed by ``to_kernel_layout``, as one kernel when the tensor is on a GPU."""
    if bWeight.is_cuda and bWeight.dim() == 4 and (bWeight.shape[1] * bWeight.shape[2]) % 32 == 0 and bWeight.shape[3] <= 8:
        return _pack_planes_cuda(bWeight, True)
    return to_kernel_layout(pack_binaryWeight(bWeight))


def pack_binaryWeight(bWeight: torch.Tensor) -> torch.Tensor:
    """``[R, n_groups, group_size, wbit]`` of +-1 -> int32 ``[R, C/32, wbit]``,
    C = n_groups*group_size, bit t of word j = (element 32*j+t == +1).
    Same contract as lut_gemm/kernel.py:9-23.  CUDA tensors are packed by a CUDA kernel."""
    if bWeight.dim() != 4:
        raise ValueError(f"BinaryWeight shape should be [N, n_groups, group_size, wbit], got {tuple(bWeight.shape)}")
    r, ng, gsz, q = bWeight.shape
    if (ng * gsz) % 32:
        raise ValueError("n_groups*group_size must be a multiple of 32")
    if bWeight.is_cuda and q <= 8 and (ng * gsz) // 32 <= 65535:
        return _pack_planes_cuda(bWeight, False)
    pos = bWeight == 1
    if not bool((pos | (bWeight == -1)).all()):
        raise ValueError("BinaryWeight should be 1 or -1, but got other values")
    return _pack_along(pos.reshape(r, ng * gsz, q), 1).contiguous()


def unpack_weight(bW: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """Dequantise: int32 ``[R, C/32, wbit]`` + alpha ``[R, G, wbit]`` -> fp32 ``[R, C]``
    with ``W[r,c] = sum_b alpha[r, c//(C/G), b] * (2*bit - 1)``, planes added in
    order b = 0, 1, ... (lut_gemm/kernel.py:26-56).  One pass per plane instead
    of the reference's G*wbit passes; results are bit-identical."""
    if bW.dim() != 3 or alpha.dim() != 3:
        raise ValueError("expected bW [R, C/32, wbit] and alpha [R, G, wbit]")
    r, w, q = bW.shape
    if alpha.shape[0] != r or alpha.shape[2] != q:
        raise ValueError("BinaryWeight and Alpha disagree on rows or number of bits")
    c, g = w * 32, alpha.shape[1]
    if c % g:
        raise ValueError("packed dimension must be divisible by the number of groups")
    out = torch.zeros(r, c, dtype=torch.float32, device=bW.device)
    a = alpha.to(torch.float32)
    for b in range(q):
        sign = _unpack_along(bW[:, :, b], 1).to(torch.float32) * 2.0 - 1.0
        out += a[:, :, b].repeat_interleave(c // g, dim=1) * sign
    return out


def unpack_to_fake_binaryWeight(packed_bweight: torch.Tensor, n_groups: int = 1) -> torch.Tensor:
    """int32 ``[R, C/32, wbit]`` -> +-1 int8 ``[R, n_groups, C/n_groups, wbit]``
    (lut_gemm/kernel.py:58-75; the reference returns uint8 where -1 reads 255)."""
    r, w, q = packed_bweight.shape
    planes = _unpack_along(packed_bweight, 1).to(torch.int8) * 2 - 1  # [R, C, q]
    return planes.reshape(r, n_groups, (w * 32) // n_groups, q)


def to_kernel_layout(packed_rows: torch.Tensor) -> torch.Tensor:
    """``[N, K/32, wbit]`` (packed along in_features) -> ``[K/32, wbit, N]``,
    the layout the kernels read (lut_gemm/quant.py:26)."""
    return packed_rows.permute(1, 2, 0).contiguous()


def convert_weight(BinaryWeight: torch.Tensor, Alpha: torch.Tensor):
    """Lat.-checkpoint tensors -> kernel tensors, for square AND non-square layers.

    ``BinaryWeight`` int32 ``[K_in, N_out/32, wbit]`` is packed along
    out_features (quant_methods/shiftaddllm.py:193-202); the result is packed
    along in_features: int32 ``[K_in/32, wbit, N_out]``.  ``Alpha [R, G, wbit]``
    becomes fp32 ``[R, wbit, G]``.  Agrees with lut_gemm/kernel.py:112-133 where
    that function works (square layers)."""
    k_in, w, q = BinaryWeight.shape
    if k_in % 32:
        raise ValueError("in_features must be a multiple of 32")
    if BinaryWeight.is_cuda and BinaryWeight.dtype == torch.int32 and q <= 8:
        from . import _lib

        src = BinaryWeight.contiguous()
        out = torch.empty((k_in // 32, q, w * 32), dtype=torch.int32, device=src.device)
        with torch.cuda.device(src.device):
            _lib.check(_lib.load().sal_repack_lat_to_kernel(src.data_ptr(), out.data_ptr(), k_in, w * 32, q,
                                                           torch.cuda.current_stream(src.device).cuda_stream),
                       "sal_repack_lat_to_kernel")
        return out, Alpha.transpose(1, 2).float().contiguous()
    bits = _unpack_along(BinaryWeight, 1)  # [K_in, N_out, q]
    repacked = _pack_along(bits, 0)        # [K_in/32, N_out, q]
    return repacked.permute(0, 2, 1).contiguous(), Alpha.transpose(1, 2).float().contiguous()


def find_layers(module, layers=(nn.Conv2d, nn.Linear), name=""):
    """Name -> module map of all leaves of the given types (lut_gemm/kernel.py:77-85)."""
    if type(module) in tuple(layers):
        return {name: module}
    found = {}
    for child_name, child in module.named_children():
        found.update(find_layers(child, layers, f"{name}.{child_name}" if name else child_name))
    return found


def _decoder_layers(model):
    """The list of decoder blocks for the model families the reference drives
    (model/opt.py, llama.py, mistral.py, gemma.py, bloom.py)."""
    inner = getattr(model, "model", None)
    if inner is not None and hasattr(inner, "decoder"):
        return inner.decoder.layers          # OPT
    if inner is not None and hasattr(inner, "layers"):
        return inner.layers                  # LLaMA / Mistral / Gemma
    if hasattr(model, "transformer") and hasattr(model.transformer, "h"):
        return model.transformer.h           # BLOOM
    raise ValueError("cannot locate the decoder layers of this model")


def _ckpt_path(weights_dir, model_name, layer_name, wbits):
    return os.path.join(weights_dir, f"{model_name}_{layer_name}_{wbits}bit.pt")


def save_lat_checkpoint(planes: torch.Tensor, alpha: torch.Tensor, weights_dir, model_name, layer_name, wbits=None,
                        invperm: torch.Tensor | None = None) -> str:
    """Writes one layer's "Lat." checkpoint file, the format the loaders below read: the step that ends
    the reference's block-wise quantisation (quant_methods/shiftaddllm.py:191-211).

    ``planes``: +-1 values ``[K_in, N_out/gs, gs, wbits]`` (one row per INPUT feature, columns in groups of
    ``gs`` outputs); ``alpha``: ``[K_in/8, N_out/gs, wbits]``, one scale per block of 8 inputs x gs outputs.
    ``invperm`` (optional, ``[K_in/8]``): with activation ordering the quantiser works on permuted blocks of
    8 input rows; this is the inverse permutation that puts blocks — of the planes and of alpha alike — back
    in model order before packing (shiftaddllm.py:195-201).
    The planes are packed along out_features with :func:`pack_binaryWeight` (on the GPU for CUDA tensors) to
    int32 ``[K_in, N_out/32, wbits]``; the file ``{weights_dir}/{model_name}_{layer_name}_{wbits}bit.pt`` holds
    ``{"bWeight": ..., "alpha": ...}`` on the CPU.  Returns the path."""
    if planes.dim() != 4 or alpha.dim() != 3:
        raise ValueError("planes must be [K_in, N_out/gs, gs, wbits] and alpha [K_in/8, N_out/gs, wbits]")
    k_in, n_group, gs, q = planes.shape
    if wbits is None:
        wbits = q
    if q != wbits:
        raise ValueError(f"Weight bit mismatch, expect {wbits} bits, but got {q} bits")
    if k_in % 8 or tuple(alpha.shape) != (k_in // 8, n_group, q):
        raise ValueError(f"alpha must be [{k_in // 8}, {n_group}, {q}], got {tuple(alpha.shape)}")
    if (n_group * gs) % 32:
        raise ValueError("out_features must be a multiple of 32")
    if invperm is not None:
        invperm = invperm.to(planes.device)
        planes = planes.reshape(k_in // 8, 8, n_group, gs, q)[invperm].reshape(k_in, n_group, gs, q)
        alpha = alpha[invperm.to(alpha.device)]
    packed = pack_binaryWeight(planes)
    os.makedirs(weights_dir, exist_ok=True)
    path = _ckpt_path(weights_dir, model_name, layer_name, wbits)
    torch.save({"bWeight": packed.cpu(), "alpha": alpha.detach().float().cpu()}, path)
    return path


def load_shiftaddllm_weight(model, weights_dir, model_name, wbits, is_lat=False):
    """Dense "simulation" load: dequantise every packed layer file into the
    ``nn.Linear`` weights (lut_gemm/kernel.py:87-109)."""
    if not is_lat:
        raise ValueError("Packed quantization weight only support lat method now")
    for i, layer in enumerate(_decoder_layers(model)):
        for name, lin in find_layers(layer).items():
            path = _ckpt_path(weights_dir, model_name, f"{i}.{name}", wbits)
            if not os.path.exists(path):
                print(f"WARNING: no such file {path}")
                continue
            ckpt = torch.load(path, map_location="cpu")
            w_t = unpack_weight(ckpt["bWeight"], ckpt["alpha"].repeat_interleave(8, dim=0))  # [K_in, N_out]
            lin.weight.data = w_t.t().contiguous().to(device=lin.weight.device, dtype=lin.weight.dtype)


def load_shiftaddllm_weight_with_kernel(model, weights_dir, model_name, wbits, is_lat=False, apot=False):
    """Swaps every decoder ``nn.Linear`` for a :class:`LutLinear` and fills it from
    the per-layer Lat. checkpoint files ``{dir}/{model}_{i}.{name}_{wbits}bit.pt``
    holding ``bWeight [K_in, N_out/32, wbit]`` and ``alpha [K_in/8, N_out/gs, wbit]``
    (lut_gemm/kernel.py:135-179).  The block alpha is kept as fp16
    ``[K_in/8, wbit, N_out/gs]`` (``apot=False``) or reduced to three int8 shifts
    as the reference does (``apot=True``)."""
    if not is_lat:
        raise ValueError("Packed quantization weight only support lat method now")
    layers = _decoder_layers(model)
    first = find_layers(layers[0])
    probe = torch.load(_ckpt_path(weights_dir, model_name, f"0.{next(iter(first))}", wbits), map_location="cpu")
    if probe["bWeight"].size(2) != wbits:
        raise ValueError(f"Weight bit mismatch, expect {wbits} bits, but got {probe['bWeight'].size(2)} bits")
    gs = (probe["bWeight"].size(1) * 32) // probe["alpha"].size(1)
    make_lut(layers, find_layers(layers), wbit=wbits, group_size=gs * 8)
    for i, layer in enumerate(_decoder_layers(model)):
        for name, lin in find_layers(layer, layers=(LutLinear,)).items():
            path = _ckpt_path(weights_dir, model_name, f"{i}.{name}", wbits)
            if not os.path.exists(path):
                print(f"WARNING: no such file {path}")
                continue
            ckpt = torch.load(path, map_location="cpu")
            bw, alpha = convert_weight(ckpt["bWeight"], ckpt["alpha"])  # [K/32,q,N], [K/8,q,N/gs]
            dev = lin.binaryWeight.device
            lin.binaryWeight = bw.to(dev)
            lin.set_block_alpha(alpha.to(dev), apot=apot)

"""``LutLinear`` and the module swappers, mirroring lut_gemm/quant.py.

Constructor and ``forward`` signatures, buffer names (``binaryWeight``,
``alpha``) and the ``[K/32, wbit, N]`` int32 packing are those of the
reference, so kernel-format state dicts load unchanged.  The dtype of
``alpha`` selects the kernel:

* fp16 ``[K/group_size, wbit, N]``            mode A, ``lutgemm_compute_shift_scale``
* fp16 ``[K/8, wbit, num_col_groups]``        mode B, ``lutgemm_compute_block``
  (``alpha_layout == "block"``)
* int8 ``[K/8, wbit, num_col_groups, 3]``     mode B, ``lutgemm_compute_block_shiftInt8``
  — the literal call of the reference's ``forward`` (lut_gemm/quant.py:50-51)

Extensions that do not break the above: ``bias=None`` works (LLaMA has no
bias), inputs may hold up to 64 rows per call (longer inputs are chunked),
and the bias add is fused into the kernel.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import lutgemm

APOT_NONE = -128


class LutLinear(nn.Module):
    def __init__(self, infeatures: int, outfeatures: int, group_size: int = 128, wbit: int = 3, bias=None):
        super().__init__()
        self.M = 1
        self.K = infeatures
        self.N = outfeatures
        self.group_size = group_size
        self.wbit = wbit
        self.num_groups = self.K // group_size
        self.num_apot = 3
        self.alpha_layout = "row"  # "row": groups along K (mode A); "block": 8 x gs blocks (mode B)
        self.register_buffer("binaryWeight", torch.zeros((self.K // 32, wbit, self.N), dtype=torch.int32))
        # same declared shape/dtype as the reference's placeholder (lut_gemm/quant.py:25)
        self.register_buffer("alpha", torch.zeros((self.N, wbit, self.num_groups, self.num_apot), dtype=torch.int8))
        self.bias = bias

    # ---- alpha setters -------------------------------------------------------------------
    def set_row_alpha(self, alpha: torch.Tensor) -> None:
        """Mode A scales ``[K/group_size, wbit, N]`` (any float dtype, stored fp16)."""
        if tuple(alpha.shape) != (self.num_groups, self.wbit, self.N):
            raise ValueError(f"row alpha must be {(self.num_groups, self.wbit, self.N)}, got {tuple(alpha.shape)}")
        self.alpha = alpha.to(torch.float16).contiguous()
        self.alpha_layout = "row"

    def set_block_alpha(self, alpha: torch.Tensor, apot: bool = False) -> None:
        """Mode B multipliers ``[K/8, wbit, N/gs]``; ``apot=True`` stores three int8 shifts."""
        if alpha.dim() != 3 or alpha.shape[0] != self.K // 8 or alpha.shape[1] != self.wbit or self.N % alpha.shape[2]:
            raise ValueError(f"block alpha must be [K/8, wbit, N/gs], got {tuple(alpha.shape)}")
        self.alpha = self.quantize_to_apot(alpha.float(), mark_missing=True) if apot else alpha.to(torch.float16).contiguous()
        self.alpha_layout = "block"

    def quantize_to_apot(self, x: torch.Tensor, mark_missing: bool = False) -> torch.Tensor:
        """alpha -> ``num_apot`` int8 power-of-two exponents (last dim).  Same
        arithmetic as lut_gemm/quant.py:30-39: each term is ``round(log2|residual|)``
        and only shifts are kept.  Where the residual is exactly zero the
        reference stores int8(-inf) = 0, a spurious 2**0; with
        ``mark_missing=True`` such terms are stored as -128, which the int8
        kernel skips."""
        terms = []
        running = torch.zeros_like(x, dtype=torch.float32)
        x = x.to(torch.float32)
        for _ in range(self.num_apot):
            resid = x - running
            shift = torch.round(torch.log(resid.abs()) / math.log(2.0))
            finite = torch.isfinite(shift)
            code = torch.where(finite, shift, torch.zeros_like(shift))
            stored = code.clamp(-128, 127).to(torch.int8)
            if mark_missing:
                stored = torch.where(finite, stored, torch.full_like(stored, APOT_NONE))
            terms.append(stored)
            running = running + torch.where(finite, torch.exp2(code) * torch.sign(resid), torch.zeros_like(code))
        return torch.stack(terms, dim=-1)

    # ---- forward -------------------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.K:
            raise RuntimeError(f"last dim of the input must be {self.K}, got {x.shape[-1]}")
        out_shape = list(x.shape[:-1]) + [self.N]
        dtype = x.dtype
        x2 = x.reshape(-1, self.K).to(torch.float16).contiguous()
        rows = x2.shape[0]
        out = torch.empty((rows, self.N), dtype=torch.float16, device=x.device)
        bias = self.bias
        if bias is not None and (bias.dtype != torch.float16 or not bias.is_contiguous()):
            bias = bias.detach().to(torch.float16).contiguous()
        for r0 in range(0, rows, lutgemm._lib.SAL_MAX_M):
            xs = x2[r0:r0 + lutgemm._lib.SAL_MAX_M]
            ys = out[r0:r0 + lutgemm._lib.SAL_MAX_M]
            self._launch(ys, xs, bias)
        return out.to(dtype).reshape(out_shape)

    def _launch(self, ys, xs, bias):
        a = self.alpha
        if a.dtype == torch.float16 and self.alpha_layout == "row":
            lutgemm.lutgemv_fused(ys, self.binaryWeight, a, bias, xs, self.N, self.K, self.wbit, a.shape[0])
            return
        if a.dtype not in (torch.float16, torch.int16, torch.int8):
            raise RuntimeError(f"unsupported alpha dtype {a.dtype}")
        # block layouts: same kernels as the reference's add-into-output entry points, with the bias
        # added by the kernel instead of a separate pre-load of the output
        lutgemm.lutgemm_block_fused(ys, self.binaryWeight, a, bias, xs, self.N, self.K, self.wbit, a.shape[2])

    def extra_repr(self):
        return "in_features={}, out_features={}, bias={}, wbit={}, group_size={}".format(
            self.K, self.N, self.bias is not None, self.wbit, self.group_size)


def make_lut(module, names, name="", wbit=3, group_size=128):
    """Replaces every attribute of ``module`` (recursively) whose dotted name is
    in ``names`` by a :class:`LutLinear` of the same shape, handing over the
    old layer's bias (lut_gemm/quant.py:63-72)."""
    if isinstance(module, LutLinear):
        return
    for child_name, child in list(module.named_children()):
        full = f"{name}.{child_name}" if name else child_name
        if full in names and not isinstance(child, LutLinear):
            new = LutLinear(child.in_features, child.out_features, group_size, wbit, bias=child.bias)
            ref = child.weight
            new.to(ref.device)
            setattr(module, child_name, new)
        else:
            make_lut(child, names, full, wbit, group_size)


def load_lut(model, checkpoint="", wbit=3, group_size=128, skip=("lm_head", "model.decoder.project_out",
                                                                 "model.decoder.project_in")):
    """Builds the skeleton (``model`` may be a HF config name/path or an
    ``nn.Module``), swaps its linear layers for :class:`LutLinear` except the
    names in ``skip``, and optionally loads a kernel-format state dict
    (lut_gemm/quant.py:74-114)."""
    if isinstance(model, str):
        import transformers

        config = transformers.AutoConfig.from_pretrained(model)
        with torch.device("meta"):
            skeleton = transformers.AutoModelForCausalLM.from_config(config, torch_dtype=torch.float16)
        model = skeleton.to_empty(device="cpu")
    model = model.eval()
    layers = {}

    def walk(mod, prefix=""):
        for child_name, child in mod.named_children():
            full = f"{prefix}.{child_name}" if prefix else child_name
            if type(child) in (nn.Linear, nn.Conv2d):
                layers[full] = child
            else:
                walk(child, full)

    walk(model)
    for name in skip:
        layers.pop(name, None)
    make_lut(model, layers, wbit=wbit, group_size=group_size)
    if checkpoint != "":
        state = torch.load(checkpoint, map_location="cpu")
        # alpha buffers change dtype/shape with the quantisation mode: adopt the stored ones
        own = dict(model.named_modules())
        for key, val in state.items():
            mod_name, _, leaf = key.rpartition(".")
            mod = own.get(mod_name)
            if isinstance(mod, LutLinear) and leaf in ("alpha", "binaryWeight"):
                setattr(mod, leaf, val.clone())
                if leaf == "alpha" and val.dtype == torch.float16 and val.dim() == 3 and val.shape[0] == mod.K // 8 \
                        and val.shape[2] != mod.N:
                    mod.alpha_layout = "block"
        model.load_state_dict(state, strict=False)
    if hasattr(model, "config") and hasattr(model.config, "max_position_embeddings"):
        model.seqlen = model.config.max_position_embeddings
    return model

"""Column-parallel partition of a BCQ linear layer over the GPUs of one node.

Output features are independent, so rank r of P keeps the columns
``[n0_r, n1_r)`` of the packed planes, of alpha and of the bias, computes its
slice of y from the full (replicated) activation vector, and the slices are
all-gathered over NCCL (NVLink).  The reference has no tensor parallelism
(its only multi-GPU code is a layer pipeline, model/opt.py:330-364).

Nothing here computes on the CPU: :class:`ColumnParallelLutLinear` wraps a
:class:`~shiftaddllm_b200.quant.LutLinear` that holds the local shard.  The
partition and gather helpers are plain tensor code and are exercised with
gloo ranks in the tests.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .quant import LutLinear

COLUMN_ALIGN = 8  # the tiled kernel moves columns in 16-byte pieces of fp16 alpha / 32-byte pieces of planes


def column_ranges(n: int, world: int, align: int = COLUMN_ALIGN) -> List[Tuple[int, int]]:
    """Contiguous, equal column ranges ``[(start, stop)] * world``.  N must split
    evenly into multiples of ``align`` so that every rank gathers the same
    number of elements (all-gather needs equal contributions)."""
    if world < 1:
        raise ValueError("world size must be positive")
    if n % world:
        raise ValueError(f"out_features {n} is not divisible by the world size {world}")
    per = n // world
    if per % align:
        raise ValueError(f"columns per rank ({per}) must be a multiple of {align}")
    return [(r * per, (r + 1) * per) for r in range(world)]


def shard_mode_a(bWeight: torch.Tensor, alpha: torch.Tensor, bias: Optional[torch.Tensor], rank: int, world: int):
    """Slices kernel-layout tensors ``bWeight [K/32,q,N]``, ``alpha [K/g,q,N]``,
    ``bias [N]`` to the columns of ``rank``."""
    n0, n1 = column_ranges(bWeight.shape[-1], world)[rank]
    b = None if bias is None else bias[n0:n1].contiguous()
    return bWeight[:, :, n0:n1].contiguous(), alpha[:, :, n0:n1].contiguous(), b


def shard_mode_b(bWeight: torch.Tensor, alpha: torch.Tensor, bias: Optional[torch.Tensor], rank: int, world: int):
    """Mode B: ``alpha [K/8,q,N/gs]`` is sliced on whole column groups."""
    n = bWeight.shape[-1]
    ngroups = alpha.shape[2]
    gs = n // ngroups
    n0, n1 = column_ranges(n, world, align=max(gs, COLUMN_ALIGN))[rank]
    b = None if bias is None else bias[n0:n1].contiguous()
    return bWeight[:, :, n0:n1].contiguous(), alpha[:, :, n0 // gs:n1 // gs].contiguous(), b


def gather_columns(y_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers ``[M, N/P]`` slices into ``[M, N]`` (rank-major columns)."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    m, n_local = y_local.shape
    flat = torch.empty((world * m, n_local), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(flat, y_local.contiguous(), group=group)  # rank r fills rows [r*m, (r+1)*m)
    buf = flat.view(world, m, n_local)
    if m == 1:
        return buf.reshape(1, world * n_local)  # already column order, no copy
    return buf.permute(1, 0, 2).reshape(m, world * n_local)


class ColumnParallelLutLinear(nn.Module):
    """A :class:`LutLinear` holding columns ``[n0, n1)`` of a layer, followed by
    an all-gather of the output slices."""

    def __init__(self, infeatures: int, outfeatures: int, group_size: int = 128, wbit: int = 3, bias=None,
                 group=None, gather_output: bool = True):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N_total = outfeatures
        self.gather_output = gather_output
        n0, n1 = column_ranges(outfeatures, self.world)[self.rank]
        self.local = LutLinear(infeatures, n1 - n0, group_size, wbit, bias=bias)

    @classmethod
    def from_full(cls, bWeight, alpha, bias, group_size: int, group=None, gather_output: bool = True):
        """Builds the local shard from full kernel-layout tensors (every rank
        holds or generates the same full tensors and keeps its slice)."""
        k = bWeight.shape[0] * 32
        q = bWeight.shape[1]
        self = cls(k, bWeight.shape[2], group_size, q, bias=None, group=group, gather_output=gather_output)
        bw, al, b = shard_mode_a(bWeight, alpha, bias, self.rank, self.world)
        self.local.binaryWeight = bw
        self.local.set_row_alpha(al)
        self.local.bias = b
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        if not self.gather_output or self.world == 1:
            return y
        lead = y.shape[:-1]
        full = gather_columns(y.reshape(-1, y.shape[-1]), self.group)
        return full.reshape(*lead, self.N_total)

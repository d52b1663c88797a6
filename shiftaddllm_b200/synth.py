"""Seeded synthetic BCQ layers with the shapes of the benchmark configurations.

Real checkpoints and datasets are not available offline; these generators
stand in for them with the value distributions the configurations state:
bit planes i.i.d. uniform +-1, alpha = 2**-k with k uniform in {2..8} (fp16,
power-of-two "Lat." scales), activations N(0,1) in fp16, bias N(0, 0.02).

All draws use CPU generators so results do not depend on the device.  Seed of
one tensor = ``base_seed*1000003 + layer_index*101 + tensor_id``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .kernel import pack_binaryWeight, to_kernel_layout

T_PLANES, T_ALPHA, T_X, T_BIAS, T_BITS = 0, 1, 2, 3, 4

# (name, K, N) of the linear layers of one decoder block
LLAMA2_7B_LINEARS = (("q_proj", 4096, 4096), ("k_proj", 4096, 4096), ("v_proj", 4096, 4096), ("o_proj", 4096, 4096),
                     ("gate_proj", 4096, 11008), ("up_proj", 4096, 11008), ("down_proj", 11008, 4096))
LLAMA2_70B_LINEARS = (("q_proj", 8192, 8192), ("k_proj", 8192, 1024), ("v_proj", 8192, 1024), ("o_proj", 8192, 8192),
                      ("gate_proj", 8192, 28672), ("up_proj", 8192, 28672), ("down_proj", 28672, 8192))
OPT_125M_QPROJ = ("q_proj", 768, 768)


def tensor_seed(base_seed: int, layer_index: int, tensor_id: int) -> int:
    return base_seed * 1000003 + layer_index * 101 + tensor_id


def _gen(base_seed, layer_index, tensor_id) -> torch.Generator:
    return torch.Generator().manual_seed(tensor_seed(base_seed, layer_index, tensor_id))


@dataclass
class BcqLayer:
    """One synthetic layer in kernel layout (CPU tensors unless moved)."""
    K: int
    N: int
    q: int
    g: int
    bWeight: torch.Tensor          # int32 [K/32, q, N]
    alpha: torch.Tensor            # fp16  [K/g, q, N]
    x: torch.Tensor                # fp16  [M, K]
    bias: Optional[torch.Tensor]   # fp16  [N] or None

    def to(self, device):
        mv = lambda t: None if t is None else t.to(device)
        return BcqLayer(self.K, self.N, self.q, self.g, mv(self.bWeight), mv(self.alpha), mv(self.x), mv(self.bias))

    def algorithmic_bytes(self) -> int:
        """Packed planes + alpha + bias + activations; the output is excluded."""
        m = self.x.shape[0]
        return (self.K * self.N * self.q // 8 + (self.K // self.g) * self.N * self.q * 2
                + (2 * self.N if self.bias is not None else 0) + 2 * m * self.K)


def make_layer(K: int, N: int, q: int = 3, g: int = 128, *, M: int = 1, bias: bool = False, base_seed: int = 0,
               layer_index: int = 0, packed_draw: bool = False) -> BcqLayer:
    """Draws one layer.  ``packed_draw=False`` draws +-1 planes ``[N, K/g, g, q]``
    and packs them with :func:`pack_binaryWeight` (the literal recipe);
    ``packed_draw=True`` draws the 32-bit words directly, which has the same
    distribution (every bit i.i.d. uniform) and is what large shapes use."""
    if K % 32 or K % g:
        raise ValueError("K must be a multiple of 32 and of the group size")
    if packed_draw:
        bw = torch.randint(-2 ** 31, 2 ** 31, (K // 32, q, N), generator=_gen(base_seed, layer_index, T_BITS),
                           dtype=torch.int64).to(torch.int32)
    else:
        planes = torch.randint(0, 2, (N, K // g, g, q), generator=_gen(base_seed, layer_index, T_PLANES),
                               dtype=torch.int8) * 2 - 1
        bw = to_kernel_layout(pack_binaryWeight(planes))
    kexp = torch.randint(2, 9, (N, K // g, q), generator=_gen(base_seed, layer_index, T_ALPHA))
    alpha = torch.exp2(-kexp.to(torch.float32)).to(torch.float16).permute(1, 2, 0).contiguous()
    x = torch.randn(M, K, generator=_gen(base_seed, layer_index, T_X)).to(torch.float16)
    b = (0.02 * torch.randn(N, generator=_gen(base_seed, layer_index, T_BIAS))).to(torch.float16) if bias else None
    return BcqLayer(K, N, q, g, bw, alpha, x, b)


def mixed_bits(num_layers: int, base_seed: int = 0) -> list:
    """Per-layer wbits from {2,3,4} with probabilities {0.3,0.5,0.2}."""
    g = torch.Generator().manual_seed(tensor_seed(base_seed, 0, 99))
    idx = torch.multinomial(torch.tensor([0.3, 0.5, 0.2]), num_layers, replacement=True, generator=g)
    return [int(2 + i) for i in idx]

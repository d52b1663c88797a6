"""The load-time packers on the GPU (include/sal_pack.h) are bit-exact with the CPU oracle,
which is pinned to the reference's own pack_binaryWeight / convert_weight outputs."""
import numpy as np
import pytest
import torch

from oracle import bcq_oracle as o
from shiftaddllm_b200 import kernel

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("r,c,q,groups", [(768, 768, 3, 6), (300, 1024, 2, 8), (4096, 4096, 3, 32), (1, 32, 1, 1),
                                          (1031, 96, 4, 3), (64, 2048, 5, 16)])
def test_pack_planes_bit_exact(r, c, q, groups):
    rng = np.random.default_rng(r + c + q)
    signs = (rng.integers(0, 2, (r, groups, c // groups, q)) * 2 - 1).astype(np.int8)
    ref = o.pack_binary_weight(signs)                                   # [R, C/32, q]
    dev = torch.from_numpy(signs).cuda()
    got = kernel.pack_binaryWeight(dev)
    assert got.dtype == torch.int32 and got.shape == ref.shape
    assert np.array_equal(got.cpu().numpy(), ref)
    assert np.array_equal(kernel.pack_binaryWeight(dev.float()).cpu().numpy(), ref)      # the reference packs float +-1 tensors
    fused = kernel.pack_to_kernel_layout(dev)                            # [C/32, q, R]
    assert np.array_equal(fused.cpu().numpy(), o.to_kernel_layout(ref))
    assert np.array_equal(kernel.pack_binaryWeight(torch.from_numpy(signs)).numpy(), ref)  # CPU path, same function


def test_pack_rejects_other_values():
    signs = torch.ones(8, 1, 64, 2, dtype=torch.int8, device="cuda")
    signs[3, 0, 17, 1] = 0
    with pytest.raises(ValueError):
        kernel.pack_binaryWeight(signs)


@pytest.mark.parametrize("k,n,q", [(768, 768, 3), (768, 3072, 3), (4096, 11008, 2), (11008, 4096, 3), (32, 32, 1), (64, 1056, 4)])
def test_lat_checkpoint_repack_bit_exact(k, n, q):
    """Checkpoint layout [K, N/32, q] (packed along output features) -> kernel layout
    [K/32, q, N], square and non-square (the reference's convert_weight only handles square)."""
    rng = np.random.default_rng(k * 7 + n + q)
    lat = rng.integers(-2 ** 31, 2 ** 31, (k, n // 32, q), dtype=np.int64).astype(np.int32)
    alpha = rng.random((k // 8, n // 16, q)).astype(np.float32)
    ref_bw, ref_alpha = o.convert_weight(lat, alpha)
    got_bw, got_alpha = kernel.convert_weight(torch.from_numpy(lat).cuda(), torch.from_numpy(alpha).cuda())
    assert np.array_equal(got_bw.cpu().numpy(), ref_bw)
    assert np.array_equal(got_alpha.cpu().numpy(), ref_alpha)
    cpu_bw, _ = kernel.convert_weight(torch.from_numpy(lat), torch.from_numpy(alpha))
    assert np.array_equal(cpu_bw.numpy(), ref_bw)

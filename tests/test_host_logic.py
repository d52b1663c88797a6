"""Host-side (CPU) logic of the product package: packers vs the reference's golden
vectors, LutLinear bookkeeping, module swapping, shard arithmetic, synthetic generators."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import bcq_oracle as o
from shiftaddllm_b200 import kernel as K
from shiftaddllm_b200 import shard, synth
from shiftaddllm_b200.quant import APOT_NONE, LutLinear, load_lut, make_lut


@pytest.mark.parametrize("tag", ["p0", "p1", "p2"])
def test_product_packers_bit_exact(golden, tag):
    planes = torch.from_numpy(golden[f"{tag}_planes"])
    packed = K.pack_binaryWeight(planes.float())
    assert packed.dtype == torch.int32 and packed.is_contiguous()
    assert torch.equal(packed, torch.from_numpy(golden[f"{tag}_packed"]))
    w = K.unpack_weight(packed, torch.from_numpy(golden[f"{tag}_alpha"]))
    assert torch.equal(w, torch.from_numpy(golden[f"{tag}_weight"]))
    fake = K.unpack_to_fake_binaryWeight(packed, planes.shape[1])
    assert torch.equal(fake, planes)


def test_pack_rejects_bad_input():
    with pytest.raises(ValueError):
        K.pack_binaryWeight(torch.zeros(2, 1, 32, 1))          # not +-1
    with pytest.raises(ValueError):
        K.pack_binaryWeight(torch.ones(2, 32, 1))              # wrong rank
    with pytest.raises(ValueError):
        K.pack_binaryWeight(torch.ones(2, 1, 16, 1))           # not a multiple of 32


def test_convert_weight(golden):
    bw, al = K.convert_weight(torch.from_numpy(golden["cv_packed_lat"]),
                              torch.from_numpy(golden["cv_alpha_blk"]).repeat_interleave(8, 0))
    assert torch.equal(bw, torch.from_numpy(golden["cv_kernel_bw"]))
    assert torch.equal(al, torch.from_numpy(golden["cv_kernel_alpha"]))
    # non-square, where the reference's function raises: compare with the oracle's converter
    g = torch.Generator().manual_seed(3)
    planes = torch.randint(0, 2, (96, 4, 16, 2), generator=g) * 2 - 1   # K_in=96, N_out=64
    lat = K.pack_binaryWeight(planes)
    alpha = torch.rand(96, 4, 2, generator=g)
    bw, al = K.convert_weight(lat, alpha)
    bw_o, al_o = o.convert_weight(lat.numpy(), alpha.numpy())
    assert bw.shape == (3, 2, 64)
    assert np.array_equal(bw.numpy(), bw_o) and np.array_equal(al.numpy(), al_o)


def test_apot(golden):
    lin = LutLinear(32, 32, 32, 3)
    got = lin.quantize_to_apot(torch.from_numpy(golden["apot_in"]))
    assert torch.equal(got, torch.from_numpy(golden["apot_out"]))
    marked = lin.quantize_to_apot(torch.tensor([0.25, 0.375]), mark_missing=True)
    assert marked[0].tolist() == [-2, APOT_NONE, APOT_NONE]
    assert marked[1].tolist() == [-1, -3, APOT_NONE]  # 0.375 = 2^-1 - 2^-3: the sign of the residual is dropped upstream


def test_lutlinear_buffers_and_state_dict():
    lin = LutLinear(256, 64, 128, 3, bias=None)
    assert lin.binaryWeight.shape == (8, 3, 64) and lin.binaryWeight.dtype == torch.int32
    assert lin.alpha.shape == (64, 3, 2, 3) and lin.alpha.dtype == torch.int8   # the reference's placeholder
    assert set(lin.state_dict()) == {"binaryWeight", "alpha"}
    lin.set_row_alpha(torch.rand(2, 3, 64))
    assert lin.alpha.dtype == torch.float16 and lin.alpha_layout == "row"
    with pytest.raises(ValueError):
        lin.set_row_alpha(torch.rand(3, 3, 64))
    lin.set_block_alpha(torch.rand(32, 3, 4), apot=True)
    assert lin.alpha.dtype == torch.int8 and lin.alpha.shape == (32, 3, 4, 3) and lin.alpha_layout == "block"
    assert "in_features=256, out_features=64" in lin.extra_repr()


def test_forward_without_gpu_raises():
    # there is no CPU path: a CPU tensor must be refused, not silently computed
    lin = LutLinear(256, 64, 128, 3)
    lin.set_row_alpha(torch.rand(2, 3, 64))
    with pytest.raises(RuntimeError):
        lin(torch.zeros(1, 256, dtype=torch.float16))


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj = nn.Linear(64, 64, bias=True)
        self.fc = nn.Sequential(nn.Linear(64, 128, bias=False), nn.ReLU(), nn.Linear(128, 64))
        self.head = nn.Linear(64, 10)


def test_make_lut_replaces_named_linears():
    blk = _Block()
    names = K.find_layers(blk)
    assert set(names) == {"q_proj", "fc.0", "fc.2", "head"}
    names.pop("head")
    old_bias = blk.q_proj.bias
    make_lut(blk, names, wbit=2, group_size=32)
    assert isinstance(blk.q_proj, LutLinear) and blk.q_proj.bias is old_bias
    assert isinstance(blk.fc[0], LutLinear) and blk.fc[0].bias is None and blk.fc[0].N == 128
    assert isinstance(blk.fc[2], LutLinear) and isinstance(blk.head, nn.Linear)
    assert blk.q_proj.wbit == 2 and blk.q_proj.num_groups == 2


def test_load_lut_state_dict_roundtrip(tmp_path):
    src = _Block()
    names = K.find_layers(src)
    names.pop("head")
    make_lut(src, names, wbit=3, group_size=32)
    for m in src.modules():
        if isinstance(m, LutLinear):
            m.binaryWeight.random_(-2 ** 31, 2 ** 31)
            m.set_row_alpha(torch.rand(m.K // 32, 3, m.N))
    path = tmp_path / "ckpt.pt"
    torch.save(src.state_dict(), path)
    dst = load_lut(_Block(), str(path), wbit=3, group_size=32, skip=("head",))
    assert torch.equal(dst.q_proj.binaryWeight, src.q_proj.binaryWeight)
    assert torch.equal(dst.fc[2].alpha, src.fc[2].alpha) and dst.fc[2].alpha.dtype == torch.float16


def test_column_ranges_and_sharding():
    assert shard.column_ranges(11008, 8) == [(i * 1376, (i + 1) * 1376) for i in range(8)]
    assert shard.column_ranges(1024, 8)[-1] == (896, 1024)
    with pytest.raises(ValueError):
        shard.column_ranges(1000, 3)
    with pytest.raises(ValueError):
        shard.column_ranges(8 * 12, 8, align=8)
    layer = synth.make_layer(256, 64, 3, 128, bias=True)
    parts = [shard.shard_mode_a(layer.bWeight, layer.alpha, layer.bias, r, 4) for r in range(4)]
    assert torch.equal(torch.cat([p[0] for p in parts], dim=2), layer.bWeight)
    assert torch.equal(torch.cat([p[1] for p in parts], dim=2), layer.alpha)
    assert torch.equal(torch.cat([p[2] for p in parts]), layer.bias)
    # every shard's product equals the matching columns of the unsharded product, bit for bit
    full = o.lutgemm_compute_shift_scale(np.zeros(64, np.float32), layer.bWeight.numpy(), layer.alpha.numpy(),
                                         layer.x.numpy())
    for r, (bw, al, _) in enumerate(parts):
        part = o.lutgemm_compute_shift_scale(np.zeros(16, np.float32), bw.numpy(), al.numpy(), layer.x.numpy())
        assert np.array_equal(part, full[16 * r:16 * (r + 1)])


def test_synth_is_seeded_and_matches_recipe():
    a = synth.make_layer(768, 768, 3, 128, bias=True)
    b = synth.make_layer(768, 768, 3, 128, bias=True)
    assert torch.equal(a.bWeight, b.bWeight) and torch.equal(a.alpha, b.alpha) and torch.equal(a.x, b.x)
    assert a.bWeight.shape == (24, 3, 768) and a.alpha.shape == (6, 3, 768) and a.x.shape == (1, 768)
    k = -torch.log2(a.alpha.float())
    assert torch.equal(k, k.round()) and k.min() >= 2 and k.max() <= 8
    assert a.algorithmic_bytes() == 251904          # the OPT-125m q_proj figure
    assert synth.make_layer(4096, 4096, 3, packed_draw=True).algorithmic_bytes() == 7086080
    c = synth.make_layer(768, 768, 3, 128, layer_index=1)
    assert not torch.equal(a.bWeight, c.bWeight)
    bits = synth.mixed_bits(224)
    assert set(bits) <= {2, 3, 4} and bits == synth.mixed_bits(224)


def test_clock_sampler_summary_uses_the_timed_window():
    """bench.ClockSampler: samples inside the marked window are the ones reported; with none inside, all samples
    since the sampler started are used and the record says so; no samples at all gives an empty record."""
    import bench

    s = bench.ClockSampler(0)
    s.source = "test"
    s.rows = [(1.0, 1200, 1965, []), (2.0, 1965, 1965, ["sw_power_cap"]), (2.5, 1950, 1965, []), (4.0, 900, 1965, ["hw_slowdown"])]
    s.t0, s.t1 = 1.5, 3.0
    rec = s.summary()
    assert rec["window"] == "timed steps" and rec["samples"] == 2 and rec["sm_mhz"] in (1950, 1957, 1965)
    assert rec["reasons"] == ["sw_power_cap"] and rec["sm_max_mhz"] == 1965
    s.t0, s.t1 = 10.0, 11.0
    rec = s.summary()
    assert rec["window"] == "warm-up and timed steps" and rec["samples"] == 4 and "hw_slowdown" in rec["reasons"]
    empty = bench.ClockSampler(0).summary()
    assert empty["samples"] == 0 and empty["sm_mhz"] is None

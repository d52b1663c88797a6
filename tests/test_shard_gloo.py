"""Column-parallel partition + all-gather with two CPU ranks over gloo.  The local
product of each rank is the oracle here (the product has no CPU compute path); what
is under test is the partition arithmetic and the gather layout."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import bcq_oracle as o
from shiftaddllm_b200 import shard, synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layer = synth.make_layer(256, 64, 3, 128, M=m, bias=True)
        bw, al, bias = shard.shard_mode_a(layer.bWeight, layer.alpha, layer.bias, rank, world)
        w_local = o.dequant_mode_a(bw.numpy(), al.numpy())
        y_local = torch.from_numpy(o.linear_fp32(layer.x.numpy(), w_local, bias.numpy())).to(torch.float16)
        y = shard.gather_columns(y_local)
        assert y.shape == (m, 64)
        torch.save(y, os.path.join(out_dir, f"y{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [1, 3])
def test_two_ranks_reassemble_the_full_output(tmp_path, m):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), m, str(tmp_path)), nprocs=world, join=True)
    layer = synth.make_layer(256, 64, 3, 128, M=m, bias=True)
    w = o.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
    full = torch.from_numpy(o.linear_fp32(layer.x.numpy(), w, layer.bias.numpy())).to(torch.float16)
    for r in range(world):
        got = torch.load(os.path.join(tmp_path, f"y{r}.pt"))
        assert torch.equal(got, full)   # sharding changes nothing, bit for bit


def test_column_parallel_decoder_shards_are_the_columns_of_one_model():
    """Host side of shiftaddllm_b200/shard_decoder.py (no GPU): every rank draws the same model and keeps its
    columns, the gather regions of the four exchange points tile the exchange buffer, and a fused exchange is
    only planned for batch 1 on more than one rank."""
    import torch

    from shiftaddllm_b200.decoder import SHAPES, BcqLlamaDecoder
    from shiftaddllm_b200.shard_decoder import ColumnParallelDecoder

    shape = SHAPES["tiny4"]
    full = BcqLlamaDecoder(shape, wbits=2, max_len=8, device="cpu", seed=4, fused=False)
    world = 4
    ranks = [ColumnParallelDecoder(shape, wbits=2, max_len=8, rank=r, world=world, device="cpu", seed=4, exchange="nccl")
             for r in range(world)]
    for name in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
        for li in range(shape.layers):
            ref = getattr(full.blocks[li], name)
            got_bw = torch.cat([getattr(r.blocks[li], name).binaryWeight for r in ranks], dim=2)
            got_alpha = torch.cat([getattr(r.blocks[li], name).alpha for r in ranks], dim=2)
            assert torch.equal(got_bw, ref.binaryWeight) and torch.equal(got_alpha, ref.alpha)
            assert all(getattr(r.blocks[li], name).N * world == ref.N for r in ranks)
    assert torch.equal(ranks[2].embed, full.embed) and torch.equal(ranks[3].blocks[1].post_norm, full.blocks[1].post_norm)
    r0 = ranks[0]
    assert not r0.fused and r0.peer is None                                   # the NCCL form was asked for
    h, kv = shape.hidden, shape.kv_heads * shape.head_dim
    assert r0.offsets == {"qkv": [0, h, h + kv], "o": [h + 2 * kv], "gu": [2 * h + 2 * kv, 2 * h + 2 * kv + shape.ffn],
                          "down": [2 * h + 2 * kv + 2 * shape.ffn]}
    assert [t.shape for t in r0.local["qkv"]] == [(1, h // world), (1, kv // world), (1, kv // world)]
    assert ColumnParallelDecoder(shape, wbits=2, max_len=8, rank=0, world=1, device="cpu", seed=4).fused is False

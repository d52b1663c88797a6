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

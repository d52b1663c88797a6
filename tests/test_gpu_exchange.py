"""Fused GEMV + all-gather epilogue, with the ranks emulated on ONE GPU: the ranks' launches are
issued one after the other on one stream and the waits come after all of them, so no kernel ever
waits for work that has not been launched.  Checked against the oracle and against the plain
grouped launch."""
import numpy as np
import pytest
import torch

from oracle import bcq_oracle as o
from shiftaddllm_b200 import _lib, lutgemm, shard, synth
from shiftaddllm_b200.exchange import PeerExchange

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_fused_exchange_assembles_full_outputs(world):
    shapes = [(1024, 2048), (1024, 512)]              # two products per launch, different widths
    layers = [synth.make_layer(k, n, 3, 128, packed_draw=True, bias=(i == 0), layer_index=i) for i, (k, n) in enumerate(shapes)]
    n_total = sum(n for _, n in shapes)
    ranks = PeerExchange.emulated(world, n_total, nslots=4)
    gather_offsets, off = [], 0
    for _, n in shapes:
        gather_offsets.append(off)
        off += n
    writers = None
    for slot in (0, 1, 0):                             # slot reuse after it was consumed
        for r, ex in enumerate(ranks):
            probs = []
            for layer in layers:
                bw, al, b = shard.shard_mode_a(layer.bWeight, layer.alpha, layer.bias, r, world)
                n_loc = bw.shape[2]
                probs.append(dict(output=torch.empty(1, n_loc, dtype=torch.float16, device="cuda"), bWeight=bw.cuda(),
                                  alpha=al.cuda(), bias=None if b is None else b.cuda(), d_input=layer.x.cuda(),
                                  mSize=n_loc, kSize=layer.K, nb=3, num_groups=layer.K // 128))
            w = ex.launch(probs, gather_offsets, slot, pdl=True)
            assert writers in (None, w) and w >= 1
            writers = w
        for ex in ranks:
            ex.wait(slot, writers)
        torch.cuda.synchronize()
        for ex in ranks:
            assert int(ex.flags[slot]) == 0            # consumed and cleared
            got = ex.buffer.float().cpu().numpy()
            for layer, goff in zip(layers, gather_offsets):
                w_full = o.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
                ref = o.linear_fp32(layer.x.numpy(), w_full, None if layer.bias is None else layer.bias.numpy())[0]
                assert o.max_rel_err(got[goff:goff + layer.N], ref) <= 1e-2
        for ex in ranks:
            ex.buffer.zero_()
    lib = _lib.load()
    ws = lutgemm.workspace_for(torch.device("cuda", torch.cuda.current_device()), 1, 8)
    assert lib.sal_workspace_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0


def test_wait_gives_up_with_a_status_instead_of_hanging():
    """A counter nobody signals: the bounded wait expires (about a second), records SAL_E_TIMEOUT in
    the workspace and the stream carries on."""
    lib = _lib.load()
    ex = PeerExchange.emulated(2, 64, nslots=2)[0]
    ex.wait(1, writers_per_rank=3)
    torch.cuda.synchronize()
    ws = lutgemm.workspace_for(torch.device("cuda", torch.cuda.current_device()), 1, 8)
    assert lib.sal_workspace_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == _lib.SAL_E_TIMEOUT
    assert lib.sal_workspace_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0   # cleared by the read

"""The column-parallel decoder (shiftaddllm_b200/shard_decoder.py) with its ranks emulated on ONE GPU: at every
exchange point all ranks' producing launches are issued before any rank's wait, so nothing ever waits for a
kernel that has not been launched.  A column-parallel decoder and a single-GPU decoder with the same seed are
the same model (same generator, same draw order, each rank keeps its columns): their logits must agree up to
the rounding of the fp16 outputs (the K splits, hence the summation order, differ between N and N/P columns)."""
import pytest
import torch

from shiftaddllm_b200 import _lib, lutgemm
from shiftaddllm_b200.decoder import SHAPES, BcqLlamaDecoder
from shiftaddllm_b200.shard_decoder import ColumnParallelDecoder, emulated, emulated_step

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
def test_emulated_ranks_match_the_single_gpu_decoder(world):
    shape = SHAPES["tiny"] if world == 2 else SHAPES["tiny4"]
    single = BcqLlamaDecoder(shape, wbits=3, group_size=128, max_len=32, seed=3, fused=True)
    ranks = emulated(shape, world, wbits=3, group_size=128, max_len=32, seed=3)
    for r in ranks:
        # every rank holds its columns of the same model
        n_loc = shape.hidden // world
        assert torch.equal(r.blocks[1].o_proj.binaryWeight, single.blocks[1].o_proj.binaryWeight[:, :, r.rank * n_loc:(r.rank + 1) * n_loc])
        r.reset()
    single.reset()
    tokens = [5, 17, 999, 3, 42, 7, 8]
    for i, t in enumerate(tokens):
        single.token.fill_(t)
        single.step()
        for r in ranks:
            r.token.fill_(t)
        emulated_step(ranks)
        torch.cuda.synchronize()
        ref = single.logits
        for r in ranks:
            assert int(r.pos) == i + 1
            err = float((r.logits[0] - ref).abs().max() / ref.abs().max())
            assert err < 2e-2, f"rank {r.rank}, step {i}: logits differ by {err}"
        # the gathered vectors are bit-identical on all ranks, so the replicated steps and the greedy token are too
        for r in ranks[1:]:
            assert torch.equal(r.logits, ranks[0].logits) and torch.equal(r.token, ranks[0].token)
            assert torch.equal(r.k_cache, ranks[0].k_cache)
    lib = _lib.load()
    ws = lutgemm.workspace_for(torch.device("cuda", torch.cuda.current_device()), 1, 8)
    assert lib.sal_workspace_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    for r in ranks:
        assert not r.peer.flags.any()                      # every counter was consumed and cleared


@pytest.mark.parametrize("batch", [1, 3])
def test_one_rank_degenerates_to_the_plain_decoder(batch):
    """world = 1 (no exchange at all), batch 1 and a lock-step batch: same logits as the single-GPU decoders."""
    from shiftaddllm_b200.decoder import BcqLlamaBatchDecoder

    shape = SHAPES["tiny"]
    single = BcqLlamaDecoder(shape, wbits=3, max_len=32, seed=2, fused=(batch == 1))
    model = ColumnParallelDecoder(shape, wbits=3, max_len=32, batch=batch, seed=2)
    prompts = torch.tensor([[5, 17, 400], [9, 2, 77], [123, 8, 31], [44, 44, 6]])[:, :batch]      # [length][batch]
    model.reset()
    model.feed(prompts.tolist())
    torch.cuda.synchronize()
    if batch == 1:
        single.reset()
        single.feed(prompts[:, 0].tolist(), chunk=1)
        assert float((model.logits[0] - single.logits).abs().max()) <= 2e-2 * float(single.logits.abs().max())
    else:
        ref = BcqLlamaBatchDecoder(shape, max_len=32, batch=batch, like=single)
        ref.reset()
        ref.feed(prompts.tolist())
        torch.cuda.synchronize()
        assert float((model.logits - ref.logits).abs().max()) <= 2e-2 * float(ref.logits.abs().max())
    model.capture()
    toks = model.generate(3)
    assert toks.shape == (3, batch)

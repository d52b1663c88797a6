"""The LLaMA-architecture decode harness on a tiny configuration: logits of every step against a
plain fp32 torch decoder that uses the dequantised weights (oracle), eager and graph-replayed."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import bcq_oracle as o
from shiftaddllm_b200.decoder import SHAPES, BcqLlamaDecoder, benchmark

pytestmark = pytest.mark.gpu


def dense(lin):
    w = o.dequant_mode_a(lin.binaryWeight.cpu().numpy(), lin.alpha.cpu().numpy())
    return torch.from_numpy(w).cuda()            # [N, K] fp32


def reference_logits(model, tokens):
    """Recomputes the whole sequence in fp32 for the last position (no cache)."""
    s = model.shape
    hd, kvh, rep = s.head_dim, s.kv_heads, s.heads // s.kv_heads
    x = model.embed[torch.tensor(tokens, device="cuda")].float()                 # [T, hidden]
    t_len = x.shape[0]
    pos = torch.arange(t_len, device="cuda")
    cos, sin = model.cos[pos], model.sin[pos]                                      # [T, hd/2]

    def rope(v, heads):
        v = v.view(t_len, heads, 2, hd // 2)
        a, b = v[:, :, 0], v[:, :, 1]
        c, s_ = cos[:, None, :], sin[:, None, :]
        return torch.stack((a * c - b * s_, b * c + a * s_), dim=2).view(t_len, heads, hd)

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + s.eps) * w.float()

    for blk in model.blocks:
        d = {k: dense(v) for k, v in blk.linears().items()}
        hn = norm(x, blk.input_norm).half().float()
        q = rope((hn @ d["q_proj"].t()).half().float(), s.heads)
        k = rope((hn @ d["k_proj"].t()).half().float(), kvh).half().float()
        v = (hn @ d["v_proj"].t()).half().float().view(t_len, kvh, hd)
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        scores = torch.einsum("thd,shd->hts", q.half().float(), k) / math.sqrt(hd)
        causal = torch.triu(torch.ones(t_len, t_len, device="cuda", dtype=torch.bool), 1)
        probs = torch.softmax(scores.masked_fill(causal, float("-inf")), dim=-1)
        attn = torch.einsum("hts,shd->thd", probs, v).reshape(t_len, s.hidden)
        x = x + (attn.half().float() @ d["o_proj"].t())
        hn = norm(x, blk.post_norm).half().float()
        act = F.silu(hn @ d["gate_proj"].t()) * (hn @ d["up_proj"].t())
        x = x + (act.half().float() @ d["down_proj"].t())
    hn = norm(x[-1:], model.final_norm)
    return (hn @ model.lm_head.float().t()).view(-1)


def test_tiny_decoder_matches_fp32_reference():
    model = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, group_size=128, max_len=32, seed=1)
    tokens = [5, 17, 999, 3, 42, 7]
    model.reset()
    for i, t in enumerate(tokens):
        model.token.fill_(t)
        model.step()
        torch.cuda.synchronize()
        ref = reference_logits(model, tokens[: i + 1])
        got = model.logits.clone()
        err = float((got - ref).abs().max() / ref.abs().max())
        assert err < 3e-2, f"step {i}: logits differ by {err}"
        assert int(model.pos) == i + 1


def test_graph_replay_equals_eager():
    model = BcqLlamaDecoder(SHAPES["tiny"], wbits=2, group_size=128, max_len=64, seed=2)
    prompt = [1, 2, 3, 4]
    model.reset()
    model.feed(prompt)
    eager = model.generate(8).cpu()
    model.capture()
    model.reset()
    model.feed(prompt)
    replayed = model.generate(8).cpu()
    assert torch.equal(eager, replayed)            # deterministic kernels: identical greedy tokens


def test_benchmark_runs():
    model = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, max_len=96, seed=3)
    res = benchmark(model, prompt_len=16, new_tokens=8, warmup=2)
    assert res["tokens_per_s"] > 0 and res["new_tokens"] == 8

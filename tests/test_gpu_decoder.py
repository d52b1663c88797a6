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


def fixed(t):
    """float tensor -> int64 fixed-point accumulator (units of 2**-32), the output format of SAL_OUT_FIXED_ATOMIC products."""
    return torch.round(t.double() * float(2 ** 32)).to(torch.int64)



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


def test_fused_helpers_match_torch():
    from shiftaddllm_b200 import decode_ops

    g = torch.Generator(device="cuda").manual_seed(0)
    n = 4096
    x = torch.randn(1, n, device="cuda", generator=g).half()
    d = torch.randn(1, n, device="cuda", generator=g).half()
    w = (1 + 0.1 * torch.randn(n, device="cuda", generator=g)).half()
    out, xo = torch.empty_like(x), torch.empty_like(x)
    decode_ops.residual_rmsnorm(x, d, w, out, xo, 1e-5)
    t = (x + d)
    ref = (t.float() * torch.rsqrt(t.float().pow(2).mean() + 1e-5) * w.float())
    assert torch.equal(xo, t) and float((out.float() - ref).abs().max()) < 4e-3
    decode_ops.residual_rmsnorm(x, None, w, out, None, 1e-5)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean() + 1e-5) * w.float()
    assert float((out.float() - ref).abs().max()) < 4e-3
    gate, up = torch.randn(11008, device="cuda", generator=g).half(), torch.randn(11008, device="cuda", generator=g).half()
    act = torch.empty_like(gate)
    decode_ops.silu_mul(gate, up, act)
    assert float((act.float() - (F.silu(gate) * up).float()).abs().max()) < 4e-3
    # rope + cache write + attention, grouped-query (8 heads on 2 kv heads)
    heads, kvh, hd, max_len, pos_v = 8, 2, 64, 40, 17
    q = torch.randn(heads * hd, device="cuda", generator=g).half()
    k = torch.randn(kvh * hd, device="cuda", generator=g).half()
    v = torch.randn(kvh * hd, device="cuda", generator=g).half()
    kc = torch.randn(max_len, kvh, hd, device="cuda", generator=g).half()
    vc = torch.randn(max_len, kvh, hd, device="cuda", generator=g).half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([pos_v], device="cuda")

    def rope(t, nh):
        t = t.view(nh, 2, hd // 2).float()
        a, b = t[:, 0], t[:, 1]
        return torch.stack((a * cos[pos_v] - b * sin[pos_v], b * cos[pos_v] + a * sin[pos_v]), 1).view(nh, hd).half()

    q_ref, k_ref = rope(q, heads), rope(k, kvh)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    kc_ref[pos_v], vc_ref[pos_v] = k_ref, v.view(kvh, hd)
    decode_ops.rope_kv_write(q, k, v, cos, sin, pos, kc, vc, heads, kvh, hd)
    assert float((q.view(heads, hd).float() - q_ref.float()).abs().max()) < 2e-3
    assert float((kc.float() - kc_ref.float()).abs().max()) < 2e-3 and torch.equal(vc, vc_ref)
    out = torch.empty(heads * hd, dtype=torch.float16, device="cuda")
    decode_ops.attention_decode(q, kc, vc, pos, out, heads, kvh, hd, 1.0 / math.sqrt(hd))
    kk = kc[: pos_v + 1].float().repeat_interleave(heads // kvh, dim=1)      # [T, heads, hd]
    vv = vc[: pos_v + 1].float().repeat_interleave(heads // kvh, dim=1)
    sc = torch.einsum("hd,thd->ht", q.view(heads, hd).float(), kk) / math.sqrt(hd)
    ref = torch.einsum("ht,thd->hd", torch.softmax(sc, -1), vv).reshape(-1)
    assert float((out.float() - ref).abs().max()) < 4e-3


@pytest.mark.parametrize("heads,kvh,hd,max_len,pos_v", [(8, 2, 64, 40, 17), (32, 32, 128, 784, 600), (64, 8, 128, 1296, 1100),
                                                        (4, 4, 32, 16, 0), (16, 2, 128, 300, 299), (8, 4, 256, 64, 33),
                                                        (8, 8, 128, 601, 600), (4, 4, 64, 203, 77),
                                                        (8, 8, 128, 4096, 3000), (32, 32, 128, 8192, 5000), (16, 2, 64, 8192, 8191)])
def test_split_attention_matches_torch(heads, kvh, hd, max_len, pos_v):
    """Attention split over the cached positions against torch, for plain and grouped-query layouts, and run twice
    on one scratch buffer (the arrival counters of the merge through L2 must have reset themselves).  Short caches
    take the cluster merge through distributed shared memory; 4096 positions on 8 kv heads the staged rows with
    the merge through L2; 8192 positions the rows read from global memory after the dependency wait."""
    from shiftaddllm_b200 import decode_ops

    g = torch.Generator(device="cuda").manual_seed(heads * 1000 + pos_v)
    q = torch.randn(heads * hd, device="cuda", generator=g).half()
    kc = torch.randn(max_len, kvh, hd, device="cuda", generator=g).half()
    vc = torch.randn(max_len, kvh, hd, device="cuda", generator=g).half()
    pos = torch.tensor([pos_v], device="cuda")
    ws = decode_ops.attention_workspace(heads, hd, "cuda")
    kk = kc[: pos_v + 1].float().repeat_interleave(heads // kvh, dim=1)
    vv = vc[: pos_v + 1].float().repeat_interleave(heads // kvh, dim=1)
    sc = torch.einsum("hd,thd->ht", q.view(heads, hd).float(), kk) / math.sqrt(hd)
    ref = torch.einsum("ht,thd->hd", torch.softmax(sc, -1), vv).reshape(-1)
    for _ in range(2):
        out = torch.zeros(heads * hd, dtype=torch.float16, device="cuda")
        decode_ops.attention_decode(q, kc, vc, pos, out, heads, kvh, hd, 1.0 / math.sqrt(hd), ws)
        assert float((out.float() - ref).abs().max()) < 4e-3
    plain = torch.empty_like(out)
    decode_ops.attention_decode(q, kc, vc, pos, plain, heads, kvh, hd, 1.0 / math.sqrt(hd))
    assert float((out.float() - plain.float()).abs().max()) < 2e-3


@pytest.mark.parametrize("heads,kvh,hd,max_len,pos_v,f32", [(8, 2, 64, 40, 17, False), (32, 32, 128, 200, 150, True),
                                                            (64, 8, 128, 300, 0, True), (8, 8, 32, 64, 63, False),
                                                            (8, 8, 128, 4096, 3000, True), (32, 32, 128, 8192, 5000, False)])
def test_rope_attention_fused_equals_two_kernels(heads, kvh, hd, max_len, pos_v, f32):
    """Rotary step + cache write + attention in one kernel against the two separate helpers:
    same cache contents and the same output; fixed-point accumulator inputs are consumed and cleared."""
    from shiftaddllm_b200 import decode_ops

    g = torch.Generator(device="cuda").manual_seed(pos_v + heads)
    q = torch.randn(heads * hd, device="cuda", generator=g)
    k = torch.randn(kvh * hd, device="cuda", generator=g)
    v = torch.randn(kvh * hd, device="cuda", generator=g)
    kc = torch.randn(max_len, kvh, hd, device="cuda", generator=g).half()
    vc = torch.randn(max_len, kvh, hd, device="cuda", generator=g).half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([pos_v], device="cuda")
    ws = decode_ops.attention_workspace(heads, hd, "cuda")
    scale = 1.0 / math.sqrt(hd)
    # two kernels
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref, out_ref = q.half(), torch.empty(heads * hd, dtype=torch.float16, device="cuda")
    decode_ops.rope_kv_write(q_ref, k.half(), v.half(), cos, sin, pos, kc_ref, vc_ref, heads, kvh, hd)
    decode_ops.attention_decode(q_ref, kc_ref, vc_ref, pos, out_ref, heads, kvh, hd, scale, ws)
    # one kernel
    qi, ki, vi = (fixed(q), fixed(k), fixed(v)) if f32 else (q.half(), k.half(), v.half())
    out = torch.empty_like(out_ref)
    assert decode_ops.rope_attention_decode(qi, ki, vi, cos, sin, pos, kc, vc, out, heads, kvh, hd, scale, ws)
    torch.cuda.synchronize()
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    assert float((out.float() - out_ref.float()).abs().max()) < 1e-3
    if f32:
        assert not qi.any() and not ki.any() and not vi.any()
    else:
        assert torch.equal(qi, q.half())          # fp16 inputs are left as they were


@pytest.mark.parametrize("n", [40, 1000, 4096, 8192, 12000])
def test_rmsnorm_helpers_all_sizes(n):
    """Register fast path (n % 8 == 0, n <= 8192) and the general path of both norm kernels against torch."""
    from shiftaddllm_b200 import decode_ops

    g = torch.Generator(device="cuda").manual_seed(n)
    x = torch.randn(1, n, device="cuda", generator=g).half()
    d = torch.randn(1, n, device="cuda", generator=g).half()
    w = (1 + 0.1 * torch.randn(n, device="cuda", generator=g)).half()
    t = x + d
    ref = t.float() * torch.rsqrt(t.float().pow(2).mean() + 1e-5) * w.float()
    out, xo = torch.empty_like(x), torch.empty_like(x)
    decode_ops.residual_rmsnorm(x, d, w, out, xo, 1e-5)
    assert torch.equal(xo, t) and float((out.float() - ref).abs().max()) < 6e-3
    d32, za = fixed(d), torch.ones(40000, dtype=torch.int64, device="cuda")
    out2, x_inplace = torch.empty_like(x), x.clone()
    decode_ops.residual_rmsnorm_fixedacc(x_inplace, d32, w, out2, x_inplace, 1e-5, za, None)
    assert torch.equal(x_inplace, t) and torch.equal(out2, out)
    assert not d32.any() and not za.any()


def test_accumulator_consuming_helpers():
    """The accumulator-consuming variants give what the fp16 helpers give on the rounded accumulator, and
    leave every accumulator they were handed at zero."""
    from shiftaddllm_b200 import decode_ops

    g = torch.Generator(device="cuda").manual_seed(3)
    n = 4096
    x = torch.randn(1, n, device="cuda", generator=g).half()
    d_f = torch.randn(1, n, device="cuda", generator=g)
    d32 = fixed(d_f)
    w = (1 + 0.1 * torch.randn(n, device="cuda", generator=g)).half()
    za, zb = torch.ones(11008, dtype=torch.int64, device="cuda"), torch.ones(300, dtype=torch.int64, device="cuda")
    out, xo = torch.empty_like(x), torch.empty_like(x)
    out_ref, xo_ref = torch.empty_like(x), torch.empty_like(x)
    decode_ops.residual_rmsnorm(x, d_f.half(), w, out_ref, xo_ref, 1e-5)
    decode_ops.residual_rmsnorm_fixedacc(x, d32, w, out, xo, 1e-5, za, zb)
    assert torch.equal(xo, xo_ref) and float((out.float() - out_ref.float()).abs().max()) < 2e-3
    assert not d32.any() and not za.any() and not zb.any()
    decode_ops.residual_rmsnorm_fixedacc(x, None, w, out, None, 1e-5)
    decode_ops.residual_rmsnorm(x, None, w, out_ref, None, 1e-5)
    assert float((out.float() - out_ref.float()).abs().max()) < 2e-3

    heads, kvh, hd, max_len, pos_v = 8, 2, 64, 40, 9
    q32 = torch.randn(heads * hd, device="cuda", generator=g)
    k32 = torch.randn(kvh * hd, device="cuda", generator=g)
    v32 = torch.randn(kvh * hd, device="cuda", generator=g)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([pos_v], device="cuda")
    kc, vc = torch.zeros(max_len, kvh, hd, device="cuda").half(), torch.zeros(max_len, kvh, hd, device="cuda").half()
    kc_ref, vc_ref = kc.clone(), vc.clone()
    q_ref, k_ref, v_ref = q32.half(), k32.half(), v32.half()
    decode_ops.rope_kv_write(q_ref, k_ref, v_ref, cos, sin, pos, kc_ref, vc_ref, heads, kvh, hd)
    q_out = torch.empty(heads * hd, dtype=torch.float16, device="cuda")
    qa, ka, va = fixed(q32), fixed(k32), fixed(v32)
    decode_ops.rope_kv_write_fixedacc(qa, ka, va, q_out, cos, sin, pos, kc, vc, heads, kvh, hd)
    assert torch.equal(q_out, q_ref) and torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    assert not qa.any() and not ka.any() and not va.any()


@pytest.mark.parametrize("mode", ["torch", "fused", "atomic"])
def test_tiny_decoder_matches_fp32_reference(mode):
    model = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, group_size=128, max_len=32, seed=1, fused=(mode != "torch"),
                            atomic=(mode == "atomic"))
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


@pytest.mark.parametrize("chunk", [64, 5])
def test_chunked_prefill_matches_token_by_token(chunk):
    """A prompt fed in chunks (every linear one small-batch product per chunk; 70 tokens = a chunk of 64 and one
    of 6, or fourteen chunks of 5) leaves the same cache, logits and next token as one decode step per token."""
    prompt = torch.randint(0, 1000, (70,), generator=torch.Generator().manual_seed(8)).tolist()
    a = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, max_len=96, seed=6)
    a.reset()
    a.feed(prompt, chunk=1)
    b = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, max_len=96, seed=6)
    b.reset()
    b.feed(prompt, chunk=chunk)
    torch.cuda.synchronize()
    assert int(a.pos) == int(b.pos) == 70
    scale = float(a.k_cache.float().abs().max())
    assert float((a.k_cache.float() - b.k_cache.float()).abs().max()) <= 2e-2 * scale
    assert float((a.v_cache.float() - b.v_cache.float()).abs().max()) <= 2e-2 * float(a.v_cache.float().abs().max())
    assert float((a.logits - b.logits).abs().max()) <= 3e-2 * float(a.logits.abs().max())
    ref = reference_logits(a, prompt)
    assert float((b.logits - ref).abs().max()) <= 3e-2 * float(ref.abs().max())
    # decoding continues from the chunk-filled cache
    tb = b.generate(4)
    assert tb.shape == (4,) and int(b.pos) == 74


def test_atomic_mode_tracks_the_deterministic_mode():
    """Fixed-point atomic accumulation only changes where the fp16 rounding happens: greedy tokens over a short
    generation agree with the fp16-output path, the accumulators are left clean, and a second run gives
    bit-identical logits (integer sums do not depend on the order in which thread blocks arrive)."""
    a = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, max_len=64, seed=4, fused=True)
    b = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, max_len=64, seed=4, fused=True, atomic=True)
    for m in (a, b):
        m.reset()
        m.feed([3, 1, 4, 1, 5])
    ta, tb = a.generate(6).cpu(), b.generate(6).cpu()
    assert torch.equal(ta, tb)
    torch.cuda.synchronize()
    for buf in (b._qacc, b._kacc, b._vacc, b._oacc, b._gateacc, b._upacc):
        assert float(buf.abs().max()) == 0.0          # consumed and cleared (down32 is cleared by the next step)
    first_logits = b.logits.clone()
    b.capture()
    b.reset()
    b.feed([3, 1, 4, 1, 5])
    assert torch.equal(b.generate(6).cpu(), ta)
    assert torch.equal(b.logits, first_logits)


def test_batch_decoder_matches_single_sequences():
    """Three sequences decoded in lock step (small-batch LUT products, M = 3) give the logits of
    the same three sequences decoded one at a time with the same weights."""
    from shiftaddllm_b200.decoder import BcqLlamaBatchDecoder

    single = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, max_len=32, seed=2, fused=False)
    batch = BcqLlamaBatchDecoder(SHAPES["tiny"], max_len=32, batch=3, like=single)
    prompts = torch.tensor([[5, 17, 400], [9, 2, 77], [123, 8, 31], [44, 44, 6]])          # [length][batch]
    batch.reset()
    batch.feed(prompts.tolist())
    torch.cuda.synchronize()
    for col in range(3):
        single.reset()
        single.feed(prompts[:, col].tolist())
        torch.cuda.synchronize()
        a, b = batch.logits[col].cpu(), single.logits.cpu()
        assert float((a - b).abs().max()) <= 2e-2 * float(b.abs().max())
        assert int(batch.token[col]) == int(single.token)
    # the M-row helpers (default) against plain torch ops between the products: same caches, same logits
    plain = BcqLlamaBatchDecoder(SHAPES["tiny"], max_len=32, batch=3, like=single, fused=False)
    plain.reset()
    plain.feed(prompts.tolist())
    torch.cuda.synchronize()
    assert float((plain.k_cache.float() - batch.k_cache.float()).abs().max()) <= 2e-2 * float(plain.k_cache.float().abs().max())
    assert float((plain.logits - batch.logits).abs().max()) <= 2e-2 * float(plain.logits.abs().max())
    batch.capture()
    toks = batch.generate(3)
    assert toks.shape == (3, 3)


@pytest.mark.parametrize("batch,heads,kvh,hd,max_len,pos_v", [(3, 8, 2, 64, 40, 17), (16, 32, 32, 128, 96, 70), (5, 64, 8, 128, 130, 0)])
def test_lock_step_helpers_match_the_single_sequence_helpers(batch, heads, kvh, hd, max_len, pos_v):
    """The batch forms of the norm and of rotary step + cache write + attention give, per sequence, exactly what
    the single-sequence helpers give."""
    from shiftaddllm_b200 import decode_ops

    g = torch.Generator(device="cuda").manual_seed(batch + heads)
    q = torch.randn(batch, heads * hd, device="cuda", generator=g).half()
    k = torch.randn(batch, kvh * hd, device="cuda", generator=g).half()
    v = torch.randn(batch, kvh * hd, device="cuda", generator=g).half()
    kc = torch.randn(batch, max_len, kvh, hd, device="cuda", generator=g).half()
    vc = torch.randn(batch, max_len, kvh, hd, device="cuda", generator=g).half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([pos_v], device="cuda")
    scale = 1.0 / math.sqrt(hd)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    out_ref = torch.empty(batch, heads * hd, dtype=torch.float16, device="cuda")
    ws1 = decode_ops.attention_workspace(heads, hd, "cuda")
    for b in range(batch):
        assert decode_ops.rope_attention_decode(q[b], k[b], v[b], cos, sin, pos, kc_ref[b], vc_ref[b], out_ref[b], heads, kvh, hd, scale, ws1)
    out = torch.empty_like(out_ref)
    ws = decode_ops.attention_workspace_batch(batch, heads, hd, "cuda")
    assert decode_ops.rope_attention_decode_batch(q, k, v, cos, sin, pos, kc, vc, out, heads, kvh, hd, scale, ws)
    torch.cuda.synchronize()
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    assert float((out.float() - out_ref.float()).abs().max()) < 2e-3      # the slices per sequence differ (fewer CTAs each)
    n = heads * hd
    x, d = q.clone(), torch.randn(batch, n, device="cuda", generator=g).half()
    w = (1 + 0.1 * torch.randn(n, device="cuda", generator=g)).half()
    o1, x1, o2, x2 = (torch.empty_like(x) for _ in range(4))
    decode_ops.residual_rmsnorm_rows(x, d, w, o1, x1, 1e-5)
    for b in range(batch):
        decode_ops.residual_rmsnorm(x[b:b + 1], d[b:b + 1], w, o2[b:b + 1], x2[b:b + 1], 1e-5)
    assert torch.equal(o1, o2) and torch.equal(x1, x2)


def test_benchmark_runs():
    model = BcqLlamaDecoder(SHAPES["tiny"], wbits=3, max_len=96, seed=3)
    res = benchmark(model, prompt_len=16, new_tokens=8, warmup=2)
    assert res["tokens_per_s"] > 0 and res["new_tokens"] == 8


@pytest.mark.parametrize("vocab", [1000, 32000, 8])
def test_greedy_token_helper(vocab):
    """fp32 copy of the logits, the first of equal maxima (as torch.argmax), position + 1; NaNs are never chosen."""
    from shiftaddllm_b200 import decode_ops

    gen = torch.Generator(device="cuda").manual_seed(vocab)
    for trial in range(4):
        lg = torch.randn(vocab, device="cuda", generator=gen).half()
        if trial == 1:      # several equal maxima, the first one not in the first thread's share
            top = lg.max() + 1
            for i in (vocab - 1, vocab // 2, vocab // 3):
                lg[i] = top
        if trial == 2:
            lg[0] = float("nan")
        if trial == 3:
            lg.fill_(-3.0)      # all equal: index 0
        out32 = torch.zeros(vocab, dtype=torch.float32, device="cuda")
        token = torch.full((1,), -1, dtype=torch.long, device="cuda")
        pos = torch.full((1,), 41, dtype=torch.long, device="cuda")
        assert decode_ops.greedy_token(lg, out32, token, pos)
        torch.cuda.synchronize()
        ref = lg.float()
        assert torch.equal(out32.nan_to_num(7.0), ref.nan_to_num(7.0))
        want = int(torch.where(ref.isnan(), torch.full_like(ref, -float("inf")), ref).argmax())
        if trial in (1, 3):
            want = vocab // 3 if trial == 1 else 0
        assert int(token) == want and int(pos) == 42
    assert not decode_ops.greedy_token(torch.zeros(12, dtype=torch.float16, device="cuda"), None, token, pos)

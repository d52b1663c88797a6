"""Batch-1 decode harness for LLaMA-architecture models whose linear layers are BCQ `LutLinear`s.

The reference wires its kernels into a decode benchmark for OPT only (`benchmark()`,
model/opt.py:366-423: 100 warm-up single-token forwards, then per-token forward + device sync,
median seconds per token).  This module is the same measurement for the LLaMA family
(model/llama.py:93-98 names the linears that get replaced): every q/k/v/o/gate/up/down
projection is a `LutLinear` (mode A), attention, RMSNorm, RoPE and `lm_head` stay in fp16
torch, as BASELINE.json's decoder configuration states.  Weights are synthetic (no checkpoints
offline): embeddings / lm_head N(0, 0.02), BCQ planes uniform +-1, alpha = 2**-k.

One decode step issues, per block: RMSNorm, ONE grouped launch for q/k/v, RoPE + cache write,
attention over a static KV cache, o_proj, RMSNorm, ONE grouped launch for gate/up, SiLU*up,
down_proj; all LUT launches use programmatic dependent launch.  The whole step (including the
greedy argmax and the position increment) is captured in a CUDA graph, so a token costs one
graph replay and no host work.

    python -m shiftaddllm_b200.decoder --model llama2-7b --prompt 512 --new 128
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
import time
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import decode_ops, lutgemm
from .quant import LutLinear


@dataclass
class LlamaShape:
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    ffn: int
    vocab: int = 32000
    rope_theta: float = 10000.0
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


SHAPES = {
    "llama2-7b": LlamaShape(4096, 32, 32, 32, 11008),
    "llama2-70b": LlamaShape(8192, 80, 64, 8, 28672),
    "tiny": LlamaShape(256, 2, 4, 2, 512, vocab=1000),
    "tiny4": LlamaShape(256, 2, 4, 4, 512, vocab=1000),    # four kv heads: splits over four ranks
}


def _synthetic_lut_linear(k, n, q, g, device, gen) -> LutLinear:
    lin = LutLinear(k, n, g, q, bias=None)
    lin.binaryWeight = torch.randint(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=torch.int32, device=device, generator=gen)
    lin.alpha = torch.exp2(-torch.randint(2, 9, (k // g, q, n), device=device, generator=gen).float()).half()
    lin.alpha_layout = "row"
    return lin


class _Block:
    def __init__(self, shape: LlamaShape, q, g, device, gen):
        h, kv = shape.hidden, shape.kv_heads * shape.head_dim
        mk = lambda k, n: _synthetic_lut_linear(k, n, q, g, device, gen)
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = mk(h, h), mk(h, kv), mk(h, kv), mk(h, h)
        self.gate_proj, self.up_proj, self.down_proj = mk(h, shape.ffn), mk(h, shape.ffn), mk(shape.ffn, h)
        self.input_norm = (1.0 + 0.02 * torch.randn(h, device=device, generator=gen)).half()
        self.post_norm = (1.0 + 0.02 * torch.randn(h, device=device, generator=gen)).half()

    def linears(self):
        return {"q_proj": self.q_proj, "k_proj": self.k_proj, "v_proj": self.v_proj, "o_proj": self.o_proj,
                "gate_proj": self.gate_proj, "up_proj": self.up_proj, "down_proj": self.down_proj}


def _group(lins, x, outs, pdl=True, x_mul=None, atomic=False, swiglu_fixed=False):
    """One grouped LUT-GEMV launch: every layer of `lins` applied to the same activation row
    (`x_mul` given: to silu(x) * x_mul, formed inside the kernel)."""
    probs = [dict(output=o, bWeight=l.binaryWeight, alpha=l.alpha, bias=l.bias, d_input=x, mSize=l.N, kSize=l.K,
                  nb=l.wbit, num_groups=l.alpha.shape[0], d_input_mul=x_mul) for l, o in zip(lins, outs)]
    lutgemm.lutgemv_grouped(probs, pdl=pdl, atomic_fixed=atomic, swiglu_fixed=swiglu_fixed)


class BcqLlamaDecoder:
    """Greedy batch-1 decoder with a static KV cache of `max_len` positions."""

    def __init__(self, shape: LlamaShape, wbits: int = 3, group_size: int = 128, max_len: int = 640, device="cuda",
                 seed: int = 0, fused: bool = True, atomic: bool = False):
        self.shape, self.max_len = shape, max_len
        self.fused = fused   # fused CUDA helpers between the GEMVs (False: plain torch ops)
        # atomic: the GEMVs add into 64-bit fixed-point accumulators with integer atomics (no split-K reduction
        # tail; integer sums do not depend on the order of arrival, so still deterministic) and the helpers
        # consume and clear those accumulators; implies fused
        self.atomic = atomic
        self.device = torch.device(device)
        gen = torch.Generator(device=self.device).manual_seed(1000003 * seed + 5)
        self.embed = (0.02 * torch.randn(shape.vocab, shape.hidden, device=self.device, generator=gen)).half()
        self.lm_head = (0.02 * torch.randn(shape.vocab, shape.hidden, device=self.device, generator=gen)).half()
        self.final_norm = (1.0 + 0.02 * torch.randn(shape.hidden, device=self.device, generator=gen)).half()
        self.blocks = [_Block(shape, wbits, group_size, self.device, gen) for _ in range(shape.layers)]
        hd, kvh = shape.head_dim, shape.kv_heads
        self.k_cache = torch.zeros(shape.layers, max_len, kvh, hd, dtype=torch.float16, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (shape.rope_theta ** (torch.arange(0, hd, 2, device=self.device).float() / hd))
        ang = torch.arange(max_len, device=self.device).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()                       # [max_len, hd/2] fp32
        self.positions = torch.arange(max_len, device=self.device)
        # static step state (graph inputs/outputs)
        self.token = torch.zeros(1, dtype=torch.long, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self.logits = torch.zeros(shape.vocab, dtype=torch.float32, device=self.device)
        h = shape.hidden
        f16 = dict(dtype=torch.float16, device=self.device)
        self._q, self._k, self._v = torch.empty(1, h, **f16), torch.empty(1, kvh * hd, **f16), torch.empty(1, kvh * hd, **f16)
        self._o, self._gate, self._up = torch.empty(1, h, **f16), torch.empty(1, shape.ffn, **f16), torch.empty(1, shape.ffn, **f16)
        self._down = torch.empty(1, h, **f16)
        self._x, self._hn = torch.empty(1, h, **f16), torch.empty(1, h, **f16)
        self._attn, self._act = torch.empty(1, h, **f16), torch.empty(1, shape.ffn, **f16)
        # fixed-point accumulators of the atomic mode (small; always present so that the mode can be switched later)
        f32 = dict(dtype=torch.int64, device=self.device)   # fixed-point accumulators, units of 2**-32
        self._qacc, self._kacc, self._vacc = torch.zeros(1, h, **f32), torch.zeros(1, kvh * hd, **f32), torch.zeros(1, kvh * hd, **f32)
        self._oacc, self._downacc = torch.zeros(1, h, **f32), torch.zeros(1, h, **f32)
        self._gateacc, self._upacc = torch.zeros(1, shape.ffn, **f32), torch.zeros(1, shape.ffn, **f32)
        self._attn_ws = decode_ops.attention_workspace(shape.heads, hd, self.device) if fused else None
        self._rope_fused = True   # rotary step inside the attention kernel (set False to run it as a kernel of its own)
        self.graph = None

    # ---- one token ------------------------------------------------------------------------
    def _rope(self, t, heads):
        hd = self.shape.head_dim
        cos = self.cos.index_select(0, self.pos)        # [1, hd/2]
        sin = self.sin.index_select(0, self.pos)
        t = t.view(heads, 2, hd // 2).float()           # rotate-half convention: (first half, second half)
        a, b = t[:, 0, :], t[:, 1, :]
        return torch.stack((a * cos - b * sin, b * cos + a * sin), dim=1).view(heads, hd).half()

    def step(self):
        """Consumes `self.token` at position `self.pos`; leaves logits, the greedy next token in
        `self.token` and `self.pos + 1` in `self.pos`.  Graph-capturable (no host sync)."""
        if self.atomic:
            return self._step_atomic()
        if self.fused:
            return self._step_fused()
        s = self.shape
        hd, kvh, rep = s.head_dim, s.kv_heads, s.heads // s.kv_heads
        x = self.embed.index_select(0, self.token)                      # [1, hidden] fp16
        mask = (self.positions > self.pos).view(1, 1, -1)               # positions not written yet
        for li, blk in enumerate(self.blocks):
            hn = F.rms_norm(x, (s.hidden,), blk.input_norm, s.eps)
            _group((blk.q_proj, blk.k_proj, blk.v_proj), hn, (self._q, self._k, self._v))
            qh = self._rope(self._q, s.heads)
            kh = self._rope(self._k, kvh)
            self.k_cache[li].index_copy_(0, self.pos, kh.view(1, kvh, hd))
            self.v_cache[li].index_copy_(0, self.pos, self._v.view(1, kvh, hd))
            keys = self.k_cache[li].permute(1, 2, 0)                    # [kvh, hd, T]
            vals = self.v_cache[li].permute(1, 0, 2)                    # [kvh, T, hd]
            scores = torch.matmul(qh.view(kvh, rep, hd), keys).float() * (1.0 / math.sqrt(hd))
            scores = scores.masked_fill(mask, float("-inf"))
            attn = torch.matmul(torch.softmax(scores, dim=-1).half(), vals).reshape(1, s.hidden)
            _group((blk.o_proj,), attn, (self._o,))
            x = x + self._o
            hn = F.rms_norm(x, (s.hidden,), blk.post_norm, s.eps)
            _group((blk.gate_proj, blk.up_proj), hn, (self._gate, self._up))
            act = F.silu(self._gate) * self._up
            _group((blk.down_proj,), act, (self._down,))
            x = x + self._down
        hn = F.rms_norm(x, (s.hidden,), self.final_norm, s.eps)
        self.logits.copy_(torch.matmul(hn, self.lm_head.t()).float().view(-1))
        self.token.copy_(self.logits.argmax().view(1))
        self.pos.add_(1)

    def _step_fused(self):
        """Same step with the fused helpers of include/sal_decode_ops.h: per block 4 LUT-GEMV
        launches + 4 helper launches (residual+RMSNorm x2, RoPE+cache write, attention); SiLU(gate)*up is
        computed inside down_proj's table build."""
        s = self.shape
        hd, kvh = s.head_dim, s.kv_heads
        scale = 1.0 / math.sqrt(hd)
        x, hn = self._x, self._hn
        torch.index_select(self.embed, 0, self.token, out=x)
        delta = None
        for li, blk in enumerate(self.blocks):
            decode_ops.residual_rmsnorm(x, delta, blk.input_norm, hn, x, s.eps)
            _group((blk.q_proj, blk.k_proj, blk.v_proj), hn, (self._q, self._k, self._v))
            if not (self._rope_fused and decode_ops.rope_attention_decode(
                    self._q, self._k, self._v, self.cos, self.sin, self.pos, self.k_cache[li], self.v_cache[li], self._attn,
                    s.heads, kvh, hd, scale, self._attn_ws)):
                decode_ops.rope_kv_write(self._q, self._k, self._v, self.cos, self.sin, self.pos, self.k_cache[li],
                                         self.v_cache[li], s.heads, kvh, hd)
                decode_ops.attention_decode(self._q, self.k_cache[li], self.v_cache[li], self.pos, self._attn, s.heads, kvh, hd,
                                            scale, self._attn_ws)
            _group((blk.o_proj,), self._attn, (self._o,))
            decode_ops.residual_rmsnorm(x, self._o, blk.post_norm, hn, x, s.eps)
            _group((blk.gate_proj, blk.up_proj), hn, (self._gate, self._up))
            _group((blk.down_proj,), self._gate, (self._down,), x_mul=self._up)   # SiLU(gate)*up formed in the table build
            delta = self._down
        decode_ops.residual_rmsnorm(x, delta, self.final_norm, hn, x, s.eps)
        self._finish(hn)

    def _finish(self, hn):
        """fp16 `lm_head` product, then fp32 logits, greedy token and position + 1 in one helper launch (torch
        operators where the helper does not take the vocabulary size)."""
        lg = torch.matmul(hn, self.lm_head.t()).view(-1)
        if not decode_ops.greedy_token(lg, self.logits, self.token, self.pos):
            self.logits.copy_(lg.float())
            self.token.copy_(self.logits.argmax().view(1))
            self.pos.add_(1)

    def set_atomic(self, atomic: bool):
        """Switches between fp16 outputs reduced in fixed order and fixed-point atomic accumulation (drops a captured graph)."""
        self.atomic = bool(atomic)
        self.graph = None
        for buf in (self._qacc, self._kacc, self._vacc, self._oacc, self._downacc, self._gateacc, self._upacc):
            buf.zero_()

    def _step_atomic(self):
        """The fused step with fixed-point atomic accumulation: every GEMV adds into an int64 buffer that starts at
        zero, the helper that consumes a buffer rounds it to fp16 and clears it again (gate/up, whose reader
        is the down projection itself, are cleared by the next residual+RMSNorm)."""
        s = self.shape
        hd, kvh = s.head_dim, s.kv_heads
        scale = 1.0 / math.sqrt(hd)
        x, hn = self._x, self._hn
        torch.index_select(self.embed, 0, self.token, out=x)
        delta = None
        for li, blk in enumerate(self.blocks):
            pend = (self._gateacc, self._upacc) if li > 0 else (None, None)
            decode_ops.residual_rmsnorm_fixedacc(x, delta, blk.input_norm, hn, x, s.eps, *pend)
            _group((blk.q_proj, blk.k_proj, blk.v_proj), hn, (self._qacc, self._kacc, self._vacc), atomic=True)
            if not (self._rope_fused and decode_ops.rope_attention_decode(
                    self._qacc, self._kacc, self._vacc, self.cos, self.sin, self.pos, self.k_cache[li], self.v_cache[li],
                    self._attn, s.heads, kvh, hd, scale, self._attn_ws)):
                decode_ops.rope_kv_write_fixedacc(self._qacc, self._kacc, self._vacc, self._q, self.cos, self.sin, self.pos,
                                                self.k_cache[li], self.v_cache[li], s.heads, kvh, hd)
                decode_ops.attention_decode(self._q, self.k_cache[li], self.v_cache[li], self.pos, self._attn, s.heads, kvh, hd,
                                            scale, self._attn_ws)
            _group((blk.o_proj,), self._attn, (self._oacc,), atomic=True)
            decode_ops.residual_rmsnorm_fixedacc(x, self._oacc, blk.post_norm, hn, x, s.eps)
            _group((blk.gate_proj, blk.up_proj), hn, (self._gateacc, self._upacc), atomic=True)
            _group((blk.down_proj,), self._gateacc, (self._downacc,), x_mul=self._upacc, atomic=True, swiglu_fixed=True)
            delta = self._downacc
        decode_ops.residual_rmsnorm_fixedacc(x, delta, self.final_norm, hn, x, s.eps, self._gateacc, self._upacc)
        self._finish(hn)

    def capture(self):
        """Captures `step` in a CUDA graph (one eager warm-up step first: it sizes the workspace and
        runs the library's one-off probes, which must not happen under capture)."""
        stream = torch.cuda.Stream(self.device)
        with torch.cuda.stream(stream):
            saved = (self.token.clone(), self.pos.clone())
            self.step()
            torch.cuda.synchronize(self.device)
            self.token.copy_(saved[0])
            self.pos.copy_(saved[1])
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                self.step()
            self.token.copy_(saved[0])
            self.pos.copy_(saved[1])
        torch.cuda.synchronize(self.device)
        self.graph, self._stream = g, stream
        return g

    def reset(self, first_token: int = 0):
        self.token.fill_(first_token)
        self.pos.zero_()
        self.k_cache.zero_()
        self.v_cache.zero_()

    def feed(self, token_ids, chunk: int = 64):
        """Teacher-forced pass over a prompt (fills the KV cache).  `chunk` > 1: the prompt goes through the
        model in chunks of up to `chunk` (at most 64) tokens, every linear layer as ONE small-batch LUT product
        per chunk — the way the reference feeds a prompt through the model's ordinary forward
        (model/opt.py:397-411) — instead of one decode step per token.  `chunk` = 1: one step (graph replay)
        per token."""
        if chunk > 1 and len(token_ids) > 1:
            return self.prefill(token_ids, chunk)
        run = self.graph.replay if self.graph is not None else self.step
        for t in token_ids:
            self.token.fill_(int(t))
            run()

    def prefill(self, token_ids, chunk: int = 64):
        """Chunked prompt pass: rows of a chunk share each weight stream (M = chunk rows per product,
        2 <= M <= 64; a last chunk of one token runs the M = 1 kernel).  RMSNorm, RoPE and the causal attention
        over the cache are torch ops here (a prompt is processed once; the per-token step is where the fused
        helpers matter).  Leaves the cache, `pos`, the logits of the last prompt token and the greedy next token
        exactly where a token-by-token `feed` would."""
        s = self.shape
        hd, kvh, rep, h = s.head_dim, s.kv_heads, s.heads // s.kv_heads, s.hidden
        chunk = max(1, min(int(chunk), 64))
        ids = torch.as_tensor(token_ids, dtype=torch.long, device=self.device).view(-1)
        p0 = int(self.pos.item())
        if p0 + ids.numel() > self.max_len:
            raise ValueError("prompt does not fit the KV cache")
        f16 = dict(dtype=torch.float16, device=self.device)
        for c0 in range(0, ids.numel(), chunk):
            tok = ids[c0:c0 + chunk]
            m = tok.numel()
            pos = torch.arange(p0 + c0, p0 + c0 + m, device=self.device)
            total = p0 + c0 + m                                            # cached positions after this chunk
            cos, sin = self.cos.index_select(0, pos)[:, None, :], self.sin.index_select(0, pos)[:, None, :]   # [m, 1, hd/2]

            def rope(t, heads):
                t = t.view(m, heads, 2, hd // 2).float()                   # rotate-half convention
                a, b = t[:, :, 0, :], t[:, :, 1, :]
                return torch.stack((a * cos - b * sin, b * cos + a * sin), dim=2).view(m, heads, hd).half()

            causal = (torch.arange(total, device=self.device)[None, :] > pos[:, None]).view(1, m, 1, total)
            x = self.embed.index_select(0, tok)                            # [m, hidden]
            q, k, v = torch.empty(m, h, **f16), torch.empty(m, kvh * hd, **f16), torch.empty(m, kvh * hd, **f16)
            o_out, down = torch.empty(m, h, **f16), torch.empty(m, h, **f16)
            gate, up = torch.empty(m, s.ffn, **f16), torch.empty(m, s.ffn, **f16)
            for li, blk in enumerate(self.blocks):
                hn = F.rms_norm(x, (h,), blk.input_norm, s.eps)
                _group((blk.q_proj, blk.k_proj, blk.v_proj), hn, (q, k, v))
                qh, kh = rope(q, s.heads), rope(k, kvh)
                self.k_cache[li].index_copy_(0, pos, kh)
                self.v_cache[li].index_copy_(0, pos, v.view(m, kvh, hd))
                keys = self.k_cache[li, :total].permute(1, 2, 0)           # [kvh, hd, T]
                vals = self.v_cache[li, :total].permute(1, 0, 2)           # [kvh, T, hd]
                scores = torch.matmul(qh.view(m, kvh, rep, hd).permute(1, 0, 2, 3), keys[:, None]).float() * (1.0 / math.sqrt(hd))
                scores = scores.masked_fill(causal, float("-inf"))         # [kvh, m, rep, T]
                attn = torch.matmul(torch.softmax(scores, dim=-1).half(), vals[:, None])       # [kvh, m, rep, hd]
                attn = attn.permute(1, 0, 2, 3).reshape(m, h).contiguous()
                _group((blk.o_proj,), attn, (o_out,))
                x = x + o_out
                hn = F.rms_norm(x, (h,), blk.post_norm, s.eps)
                _group((blk.gate_proj, blk.up_proj), hn, (gate, up))
                _group((blk.down_proj,), gate, (down,), x_mul=up)          # SiLU(gate)*up formed in the table build
                x = x + down
        hn = F.rms_norm(x[-1:], (h,), self.final_norm, s.eps)
        self.logits.copy_(torch.matmul(hn, self.lm_head.t()).float().view(-1))
        self.token.copy_(self.logits.argmax().view(1))
        self.pos.add_(ids.numel())

    def generate(self, n):
        run = self.graph.replay if self.graph is not None else self.step
        out = []
        for _ in range(n):
            run()
            out.append(self.token.clone())
        return torch.cat(out)


class BcqLlamaBatchDecoder:
    """Greedy decoder for `batch` sequences that advance in lock step (one shared position counter, as in a
    benchmark where all prompts have the same length).  The linear layers run as ONE small-batch LUT product
    per group (M = batch: the weights are streamed once for all sequences); the steps between them are the
    M-row forms of the fused helpers (residual + RMSNorm per row, rotary step + cache write + split attention
    per sequence in one launch) or, with `fused=False`, plain torch ops.  Weights are those of a
    `BcqLlamaDecoder` (pass it as `like` to share them instead of drawing new ones)."""

    def __init__(self, shape: LlamaShape, wbits: int = 3, group_size: int = 128, max_len: int = 640, batch: int = 16,
                 device="cuda", seed: int = 0, like: "BcqLlamaDecoder | None" = None, fused: bool = True):
        if not 1 <= batch <= 64:
            raise ValueError("batch must be 1..64 (rows of one small-batch LUT product)")
        self.shape, self.max_len, self.batch = shape, max_len, batch
        self.device = torch.device(device)
        if like is None:
            like = BcqLlamaDecoder(shape, wbits, group_size, max_len=8, device=device, seed=seed, fused=False)
        self.embed, self.lm_head, self.final_norm, self.blocks = like.embed, like.lm_head, like.final_norm, like.blocks
        hd, kvh, h, b = shape.head_dim, shape.kv_heads, shape.hidden, batch
        self.k_cache = torch.zeros(shape.layers, b, max_len, kvh, hd, dtype=torch.float16, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        inv = 1.0 / (shape.rope_theta ** (torch.arange(0, hd, 2, device=self.device).float() / hd))
        ang = torch.arange(max_len, device=self.device).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.positions = torch.arange(max_len, device=self.device)
        self.token = torch.zeros(b, dtype=torch.long, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self.logits = torch.zeros(b, shape.vocab, dtype=torch.float32, device=self.device)
        f16 = dict(dtype=torch.float16, device=self.device)
        self._q, self._k, self._v = torch.empty(b, h, **f16), torch.empty(b, kvh * hd, **f16), torch.empty(b, kvh * hd, **f16)
        self._o, self._down = torch.empty(b, h, **f16), torch.empty(b, h, **f16)
        self._gate, self._up = torch.empty(b, shape.ffn, **f16), torch.empty(b, shape.ffn, **f16)
        self._x, self._hn, self._attn = torch.empty(b, h, **f16), torch.empty(b, h, **f16), torch.empty(b, h, **f16)
        self.fused = fused
        self._attn_ws = decode_ops.attention_workspace_batch(b, shape.heads, hd, self.device) if fused else None
        self.graph = None

    def _rope(self, t, heads):
        hd, b = self.shape.head_dim, self.batch
        cos = self.cos.index_select(0, self.pos)        # [1, hd/2], the same position for every sequence
        sin = self.sin.index_select(0, self.pos)
        t = t.view(b, heads, 2, hd // 2).float()
        a, c = t[:, :, 0, :], t[:, :, 1, :]
        return torch.stack((a * cos - c * sin, c * cos + a * sin), dim=2).view(b, heads, hd).half()

    def _step_fused(self):
        """The step with the M-row helpers: per block 4 small-batch LUT launches + 3 helper launches."""
        s = self.shape
        hd, kvh = s.head_dim, s.kv_heads
        scale = 1.0 / math.sqrt(hd)
        x, hn = self._x, self._hn
        torch.index_select(self.embed, 0, self.token, out=x)
        delta = None
        for li, blk in enumerate(self.blocks):
            decode_ops.residual_rmsnorm_rows(x, delta, blk.input_norm, hn, x, s.eps)
            _group((blk.q_proj, blk.k_proj, blk.v_proj), hn, (self._q, self._k, self._v))
            if not decode_ops.rope_attention_decode_batch(self._q, self._k, self._v, self.cos, self.sin, self.pos, self.k_cache[li],
                                                          self.v_cache[li], self._attn, s.heads, kvh, hd, scale, self._attn_ws):
                raise RuntimeError("this head shape is not taken by the fused attention helper: use fused=False")
            _group((blk.o_proj,), self._attn, (self._o,))
            decode_ops.residual_rmsnorm_rows(x, self._o, blk.post_norm, hn, x, s.eps)
            _group((blk.gate_proj, blk.up_proj), hn, (self._gate, self._up))
            _group((blk.down_proj,), self._gate, (self._down,), x_mul=self._up)   # SiLU(gate)*up formed in the table build
            delta = self._down
        decode_ops.residual_rmsnorm_rows(x, delta, self.final_norm, hn, x, s.eps)
        self.logits.copy_(torch.matmul(hn, self.lm_head.t()).float())
        self.token.copy_(self.logits.argmax(dim=-1))
        self.pos.add_(1)

    def step(self):
        if self.fused:
            return self._step_fused()
        s, b = self.shape, self.batch
        hd, kvh, rep = s.head_dim, s.kv_heads, s.heads // s.kv_heads
        x = self.embed.index_select(0, self.token)                      # [b, hidden]
        mask = (self.positions > self.pos).view(1, 1, 1, -1)
        for li, blk in enumerate(self.blocks):
            hn = F.rms_norm(x, (s.hidden,), blk.input_norm, s.eps)
            _group((blk.q_proj, blk.k_proj, blk.v_proj), hn, (self._q, self._k, self._v))
            qh, kh = self._rope(self._q, s.heads), self._rope(self._k, kvh)
            self.k_cache[li].index_copy_(1, self.pos, kh.view(b, 1, kvh, hd))
            self.v_cache[li].index_copy_(1, self.pos, self._v.view(b, 1, kvh, hd))
            keys = self.k_cache[li].permute(0, 2, 3, 1)                 # [b, kvh, hd, T]
            vals = self.v_cache[li].permute(0, 2, 1, 3)                 # [b, kvh, T, hd]
            scores = torch.matmul(qh.view(b, kvh, rep, hd), keys).float() * (1.0 / math.sqrt(hd))
            scores = scores.masked_fill(mask, float("-inf"))
            attn = torch.matmul(torch.softmax(scores, dim=-1).half(), vals).reshape(b, s.hidden)
            _group((blk.o_proj,), attn, (self._o,))
            x = x + self._o
            hn = F.rms_norm(x, (s.hidden,), blk.post_norm, s.eps)
            _group((blk.gate_proj, blk.up_proj), hn, (self._gate, self._up))
            _group((blk.down_proj,), self._gate, (self._down,), x_mul=self._up)   # SiLU(gate)*up formed in the table build
            x = x + self._down
        hn = F.rms_norm(x, (s.hidden,), self.final_norm, s.eps)
        self.logits.copy_(torch.matmul(hn, self.lm_head.t()).float())
        self.token.copy_(self.logits.argmax(dim=-1))
        self.pos.add_(1)

    capture = BcqLlamaDecoder.capture
    generate_step = step

    def reset(self):
        self.token.zero_()
        self.pos.zero_()
        self.k_cache.zero_()
        self.v_cache.zero_()

    def feed(self, token_rows):
        """Teacher-forced pass over prompts of equal length: `token_rows` [length][batch] token ids."""
        run = self.graph.replay if self.graph is not None else self.step
        for row in token_rows:
            self.token.copy_(torch.as_tensor(row, dtype=torch.long, device=self.device))
            run()

    def generate(self, n):
        run = self.graph.replay if self.graph is not None else self.step
        out = []
        for _ in range(n):
            run()
            out.append(self.token.clone())
        return torch.stack(out)                                          # [n, batch]


def benchmark_batch(model: BcqLlamaBatchDecoder, prompt_len: int, new_tokens: int, warmup: int = 5, seed: int = 0):
    """Aggregate tokens/s of `model.batch` sequences decoded in lock step (wall clock over the new
    tokens, one device sync at the end), after prompts of `prompt_len` uniform random ids."""
    dev = model.device
    gen = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, model.shape.vocab, (prompt_len, model.batch), generator=gen)
    if model.graph is None:
        model.capture()
    model.reset()
    model.feed(prompts)
    torch.cuda.synchronize(dev)
    state = (model.token.clone(), model.pos.clone())
    for _ in range(warmup):
        model.graph.replay()
    model.token.copy_(state[0])
    model.pos.copy_(state[1])
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for _ in range(new_tokens):
        model.graph.replay()
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    return {"tokens_per_s": model.batch * new_tokens / wall, "ms_per_step": 1e3 * wall / new_tokens, "batch": model.batch,
            "prompt_len": prompt_len, "new_tokens": new_tokens}


def benchmark(model: BcqLlamaDecoder, prompt_len: int, new_tokens: int, warmup: int = 10, seed: int = 0):
    """tokens/s over `new_tokens` greedy decode steps after a `prompt_len`-token prompt of uniform
    random ids (wall clock, one device sync at the end), plus the reference-style median of
    per-token latencies measured with a sync per token (model/opt.py:405-421)."""
    dev = model.device
    gen = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, model.shape.vocab, (prompt_len,), generator=gen).tolist()
    if model.graph is None:
        model.capture()
    model.reset()
    model.feed(prompt)
    torch.cuda.synchronize(dev)
    state = (model.token.clone(), model.pos.clone())
    for _ in range(warmup):                      # warm-up replays on the real cache, then rewind
        model.graph.replay()
    model.token.copy_(state[0])
    model.pos.copy_(state[1])
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for _ in range(new_tokens):
        model.graph.replay()
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    model.token.copy_(state[0])
    model.pos.copy_(state[1])
    lat = []
    for _ in range(new_tokens):
        t1 = time.perf_counter()
        model.graph.replay()
        torch.cuda.synchronize(dev)
        lat.append(time.perf_counter() - t1)
    return {"tokens_per_s": new_tokens / wall, "ms_per_token": 1e3 * wall / new_tokens,
            "median_ms_per_token_synced": 1e3 * statistics.median(lat), "prompt_len": prompt_len, "new_tokens": new_tokens}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama2-7b", choices=sorted(SHAPES))
    ap.add_argument("--wbits", type=int, default=3)
    ap.add_argument("--groupsize", type=int, default=128)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--no-fused", action="store_true", help="plain torch ops between the GEMVs")
    ap.add_argument("--atomic", action="store_true", help="GEMVs accumulate into fixed-point buffers with integer atomics (no split-K tail, still deterministic)")
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded in lock step (small-batch LUT products)")
    args = ap.parse_args()
    shape = SHAPES[args.model]
    if args.batch > 1:
        model = BcqLlamaBatchDecoder(shape, args.wbits, args.groupsize, max_len=args.prompt + 2 * args.new + 16, batch=args.batch)
        res = benchmark_batch(model, args.prompt, args.new)
        res.update({"model": args.model, "wbits": args.wbits, "groupsize": args.groupsize, "data": "synthetic weights and prompts"})
        print(json.dumps(res))
        return
    model = BcqLlamaDecoder(shape, args.wbits, args.groupsize, max_len=args.prompt + 2 * args.new + 16, fused=not args.no_fused,
                            atomic=args.atomic)
    res = benchmark(model, args.prompt, args.new)
    res.update({"atomic_fixed_outputs": args.atomic, "fused_helpers": not args.no_fused, "model": args.model, "wbits": args.wbits, "groupsize": args.groupsize, "data": "synthetic weights and prompt"})
    print(json.dumps(res))


if __name__ == "__main__":
    main()

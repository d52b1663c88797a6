"""Column-parallel decode harness: a LLaMA-architecture decoder whose BCQ linear layers are split by
output columns over the GPUs of one node, one process per GPU.

The reference's only multi-GPU code is a layer pipeline (`opt_multigpu`, model/opt.py:330-364, driven by
`benchmark()`, model/opt.py:366-423); this is the tensor-parallel replacement the sharding of the LUT-GEMV
path calls for.  Rank r keeps columns [r*N/P, (r+1)*N/P) of every projection (packed planes, alpha), every
rank holds the full activation vector, and the [1, N/P] output slices of a launch are all-gathered:

* batch 1, ``exchange="fused"``: the gather is part of the GEMV kernel (`sal_lutgemv_grouped_exchange`: the
  CTA that finishes an output element stores it into every rank's gather buffer over NVLink and counts in),
  followed by the one-thread wait kernel.  Four exchange points per decoder block: q/k/v, o, gate/up, down.
* ``exchange="nccl"`` (and any batch > 1): the product writes its local slice, NCCL all-gathers.

Everything between the products is replicated (every rank computes RMSNorm, RoPE and attention over the
full vectors: the gathered buffers are bit-identical on all ranks, so all ranks pick the same greedy token
without another exchange); the KV cache and the fp16 ``lm_head`` are replicated too.  Attention does not get
faster with more GPUs in this arrangement — the per-token step is bound by the latency of its exchange
points, not by bandwidth.

Weights are synthetic and drawn exactly as `decoder.BcqLlamaDecoder` draws them (same generator, same
order), each rank keeping its columns: a column-parallel decoder and a single-GPU decoder with the same
seed are the same model, which is how the tests check one against the other.  With ranks emulated on one
GPU (`emulated`), the ranks' launches of one exchange point are issued one after the other before any of
their waits, so no kernel ever waits for a kernel that has not been launched.
"""
from __future__ import annotations

import math
import time
from typing import List

import torch
import torch.nn.functional as F

from . import decode_ops, lutgemm
from .decoder import LlamaShape, _synthetic_lut_linear
from .exchange import PeerExchange
from .shard import column_ranges

NSLOTS = 4


def _shard_linear(lin, rank, world):
    """Keeps the columns of `rank` of a freshly drawn full layer."""
    n0, n1 = column_ranges(lin.N, world)[rank]
    bw = lin.binaryWeight[:, :, n0:n1].contiguous()
    alpha = lin.alpha[:, :, n0:n1].contiguous()
    lin.binaryWeight, lin.alpha = bw, alpha
    lin.N_full, lin.N = lin.N, n1 - n0
    return lin


class _ShardedBlock:
    NAMES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")

    def __init__(self, shape: LlamaShape, q, g, device, gen, rank, world):
        h, kv = shape.hidden, shape.kv_heads * shape.head_dim
        dims = {"q_proj": (h, h), "k_proj": (h, kv), "v_proj": (h, kv), "o_proj": (h, h), "gate_proj": (h, shape.ffn),
                "up_proj": (h, shape.ffn), "down_proj": (shape.ffn, h)}
        for name in self.NAMES:     # same draw order as decoder._Block
            k, n = dims[name]
            setattr(self, name, _shard_linear(_synthetic_lut_linear(k, n, q, g, device, gen), rank, world))
        self.input_norm = (1.0 + 0.02 * torch.randn(h, device=device, generator=gen)).half()
        self.post_norm = (1.0 + 0.02 * torch.randn(h, device=device, generator=gen)).half()


class ColumnParallelDecoder:
    """Greedy decoder for `batch` sequences in lock step on `world` GPUs (this process is rank `rank`)."""

    def __init__(self, shape: LlamaShape, wbits: int = 2, group_size: int = 128, max_len: int = 1280, batch: int = 1,
                 rank: int = 0, world: int = 1, device="cuda", seed: int = 0, exchange: str = "fused", peer: PeerExchange | None = None,
                 group=None):
        if world < 1 or not 1 <= batch <= 64:
            raise ValueError("world must be positive and batch 1..64")
        self.shape, self.max_len, self.batch, self.rank, self.world, self.group = shape, max_len, batch, rank, world, group
        self.device = torch.device(device)
        self.fused = world > 1 and batch == 1 and exchange == "fused"
        gen = torch.Generator(device=self.device).manual_seed(1000003 * seed + 5)
        self.embed = (0.02 * torch.randn(shape.vocab, shape.hidden, device=self.device, generator=gen)).half()
        self.lm_head = (0.02 * torch.randn(shape.vocab, shape.hidden, device=self.device, generator=gen)).half()
        self.final_norm = (1.0 + 0.02 * torch.randn(shape.hidden, device=self.device, generator=gen)).half()
        self.blocks = [_ShardedBlock(shape, wbits, group_size, self.device, gen, rank, world) for _ in range(shape.layers)]
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
        kv = kvh * hd
        # full-width vectors every rank ends up with, per exchange point: [q | k | v], [o], [gate | up], [down]
        self.widths = {"qkv": (h, kv, kv), "o": (h,), "gu": (shape.ffn, shape.ffn), "down": (h,)}
        total = sum(sum(w) for w in self.widths.values())
        if self.fused:
            self.peer = peer if peer is not None else PeerExchange.symmetric(total, nslots=NSLOTS, group=group)
            store = self.peer.buffer
        else:
            self.peer = None
            store = torch.zeros(b * total, **f16)
        self.full, self.offsets, off = {}, {}, 0
        for key, ws in self.widths.items():
            views, offs = [], []
            for w in ws:
                views.append(store[off:off + b * w].view(b, w))
                offs.append(off)
                off += b * w
            self.full[key], self.offsets[key] = views, offs
        # local output slices
        self.local = {key: [torch.empty(b, w // world, **f16) for w in ws] for key, ws in self.widths.items()}
        self._x, self._hn = torch.empty(b, h, **f16), torch.empty(b, h, **f16)
        self._attn, self._act = torch.empty(b, h, **f16), torch.empty(b, shape.ffn, **f16)
        self._attn_ws = (decode_ops.attention_workspace(shape.heads, hd, self.device) if batch == 1
                         else decode_ops.attention_workspace_batch(batch, shape.heads, hd, self.device))
        self._launches = None
        self._slot = 0
        self.graph = None

    # ---- launches ---------------------------------------------------------------------------
    def _problems(self, lins, x, outs):
        return [dict(output=o, bWeight=l.binaryWeight, alpha=l.alpha, bias=None, d_input=x, mSize=l.N, kSize=l.K, nb=l.wbit,
                     num_groups=l.alpha.shape[0]) for l, o in zip(lins, outs)]

    def _prepare(self):
        """One prepared launch per (block, exchange point): validated, planned and marshalled once."""
        self._launches = []
        for blk in self.blocks:
            per = {}
            for key, lins, x in (("qkv", (blk.q_proj, blk.k_proj, blk.v_proj), self._hn), ("o", (blk.o_proj,), self._attn),
                                 ("gu", (blk.gate_proj, blk.up_proj), self._hn), ("down", (blk.down_proj,), self._act)):
                probs = self._problems(lins, x, self.local[key])
                if self.fused:
                    per[key] = self.peer.prepare(probs, self.offsets[key], pdl=True)
                else:
                    per[key] = lutgemm.prepare_grouped(probs, pdl=True)
            self._launches.append(per)

    def _product(self, li, key):
        """Generator: issues the product of exchange point `key` of block `li` and gathers its slices; yields once,
        between the producing launch and the wait for the other ranks (where an emulation switches ranks)."""
        launch = self._launches[li][key]
        if self.fused:
            slot = self._slot
            self._slot = (self._slot + 1) % NSLOTS
            launch(slot)
            yield
            self.peer.wait(slot, launch.writers)
            return
        launch()
        if self.world > 1:
            import torch.distributed as dist

            b = self.batch
            for loc, full in zip(self.local[key], self.full[key]):
                n_loc = loc.shape[1]
                flat = torch.empty((self.world * b, n_loc), dtype=loc.dtype, device=loc.device)
                dist.all_gather_into_tensor(flat, loc, group=self.group)          # rank r fills rows [r*b, (r+1)*b)
                full.copy_(flat.view(self.world, b, n_loc).permute(1, 0, 2).reshape(b, self.world * n_loc))
        else:
            for loc, full in zip(self.local[key], self.full[key]):
                full.copy_(loc)
        yield

    # ---- one token ----------------------------------------------------------------------------
    def _rope(self, t, heads):
        hd, b = self.shape.head_dim, self.batch
        cos = self.cos.index_select(0, self.pos)
        sin = self.sin.index_select(0, self.pos)
        t = t.reshape(b, heads, 2, hd // 2).float()
        a, c = t[:, :, 0, :], t[:, :, 1, :]
        return torch.stack((a * cos - c * sin, c * cos + a * sin), dim=2).view(b, heads, hd).half()

    def _phases(self):
        s, b = self.shape, self.batch
        hd, kvh, rep, h = s.head_dim, s.kv_heads, s.heads // s.kv_heads, s.hidden
        scale = 1.0 / math.sqrt(hd)
        if self._launches is None:
            self._prepare()
        x, hn = self._x, self._hn
        torch.index_select(self.embed, 0, self.token, out=x)
        q, k, v = self.full["qkv"]
        (o_full,), (gate, up), (down,) = self.full["o"], self.full["gu"], self.full["down"]
        delta = None
        mask = (self.positions > self.pos).view(1, 1, 1, -1) if b > 1 else None
        for li, blk in enumerate(self.blocks):
            if b == 1:
                decode_ops.residual_rmsnorm(x, delta, blk.input_norm, hn, x, s.eps)
            else:
                decode_ops.residual_rmsnorm_rows(x, delta, blk.input_norm, hn, x, s.eps)
            yield from self._product(li, "qkv")
            if b == 1:
                if not decode_ops.rope_attention_decode(q, k, v, self.cos, self.sin, self.pos, self.k_cache[li, 0], self.v_cache[li, 0],
                                                        self._attn, s.heads, kvh, hd, scale, self._attn_ws):
                    decode_ops.rope_kv_write(q, k, v, self.cos, self.sin, self.pos, self.k_cache[li, 0], self.v_cache[li, 0],
                                             s.heads, kvh, hd)
                    decode_ops.attention_decode(q, self.k_cache[li, 0], self.v_cache[li, 0], self.pos, self._attn, s.heads, kvh, hd,
                                                scale, self._attn_ws)
            elif not decode_ops.rope_attention_decode_batch(q, k, v, self.cos, self.sin, self.pos, self.k_cache[li], self.v_cache[li],
                                                            self._attn, s.heads, kvh, hd, scale, self._attn_ws):
                qh, kh = self._rope(q, s.heads), self._rope(k, kvh)       # head shapes the fused helper does not take
                self.k_cache[li].index_copy_(1, self.pos, kh.view(b, 1, kvh, hd))
                self.v_cache[li].index_copy_(1, self.pos, v.reshape(b, 1, kvh, hd))
                keys = self.k_cache[li].permute(0, 2, 3, 1)
                vals = self.v_cache[li].permute(0, 2, 1, 3)
                scores = torch.matmul(qh.view(b, kvh, rep, hd), keys).float() * scale
                scores = scores.masked_fill(mask, float("-inf"))
                self._attn.copy_(torch.matmul(torch.softmax(scores, dim=-1).half(), vals).reshape(b, h))
            yield from self._product(li, "o")
            if b == 1:
                decode_ops.residual_rmsnorm(x, o_full, blk.post_norm, hn, x, s.eps)
            else:
                decode_ops.residual_rmsnorm_rows(x, o_full, blk.post_norm, hn, x, s.eps)
            yield from self._product(li, "gu")
            if b == 1:
                decode_ops.silu_mul(gate, up, self._act)
            else:
                decode_ops.silu_mul(gate, up, self._act)
            yield from self._product(li, "down")
            delta = down
        if b == 1:
            decode_ops.residual_rmsnorm(x, delta, self.final_norm, hn, x, s.eps)
        else:
            decode_ops.residual_rmsnorm_rows(x, delta, self.final_norm, hn, x, s.eps)
        self.logits.copy_(torch.matmul(hn, self.lm_head.t()).float())
        self.token.copy_(self.logits.argmax(dim=-1))
        self.pos.add_(1)

    def step(self):
        """Consumes `self.token` at `self.pos`; leaves logits, the greedy next tokens and `pos + 1`.  Graph-capturable."""
        for _ in self._phases():
            pass

    def capture(self):
        """Captures `step` in a CUDA graph (after one eager warm-up step, which sizes the scratch buffers and
        runs the library's one-off probes; all ranks must call this together)."""
        stream = torch.cuda.Stream(self.device)
        with torch.cuda.stream(stream):
            saved = (self.token.clone(), self.pos.clone(), self._slot)
            self.step()
            torch.cuda.synchronize(self.device)
            self.token.copy_(saved[0])
            self.pos.copy_(saved[1])
            # a step uses 4 exchange points per block: the counter slots line up again after every step
            assert (4 * len(self.blocks)) % NSLOTS == 0 and self._slot == saved[2]
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

    def feed(self, token_rows):
        """Teacher-forced pass over prompts of equal length: `token_rows` [length][batch] (or [length] for batch 1)."""
        run = self.graph.replay if self.graph is not None else self.step
        for row in token_rows:
            self.token.copy_(torch.as_tensor(row, dtype=torch.long, device=self.device).view(-1))
            run()

    def generate(self, n):
        run = self.graph.replay if self.graph is not None else self.step
        out = []
        for _ in range(n):
            run()
            out.append(self.token.clone())
        return torch.stack(out)                                          # [n, batch]


def emulated(shape: LlamaShape, world: int, **kwargs) -> List[ColumnParallelDecoder]:
    """All ranks of a batch-1 column-parallel decoder on ONE GPU (tests): returns the rank objects; drive them
    with `emulated_step`."""
    h, kv = shape.hidden, shape.kv_heads * shape.head_dim
    total = h + 2 * kv + h + 2 * shape.ffn + h            # [q | k | v], [o], [gate | up], [down]
    peers = PeerExchange.emulated(world, total, NSLOTS, device=kwargs.get("device", "cuda"))
    return [ColumnParallelDecoder(shape, rank=r, world=world, peer=peers[r], exchange="fused", **kwargs) for r in range(world)]


def emulated_step(ranks: List[ColumnParallelDecoder]):
    """One token on all emulated ranks: at every exchange point all ranks issue their producing launch before
    any rank enqueues its wait."""
    gens = [r._phases() for r in ranks]
    done = [False] * len(gens)
    while not all(done):
        for i, g in enumerate(gens):
            if not done[i]:
                try:
                    next(g)
                except StopIteration:
                    done[i] = True


def benchmark(model: ColumnParallelDecoder, prompt_len: int, new_tokens: int, warmup: int = 3, seed: int = 0):
    """Aggregate tokens/s over `new_tokens` greedy steps after a `prompt_len`-token prompt of uniform random ids
    (the same ids on every rank).  Timed on the device (CUDA events around the graph replays); the caller takes
    the maximum over ranks."""
    dev = model.device
    gen = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, model.shape.vocab, (prompt_len, model.batch), generator=gen)
    if model.graph is None:
        model.capture()
    model.reset()
    model.feed(prompts)
    torch.cuda.synchronize(dev)
    return benchmark_steps(model, new_tokens, warmup, prompt_len)


def benchmark_steps(model: ColumnParallelDecoder, new_tokens: int, warmup: int = 3, prompt_len: int | None = None):
    """Times `new_tokens` graph replays from the current cache state (CUDA events on the replay stream)."""
    dev = model.device
    if model.graph is None:
        model.capture()
    if prompt_len is None:
        prompt_len = int(model.pos.item())
    state = (model.token.clone(), model.pos.clone())
    for _ in range(warmup):
        model.graph.replay()
    model.token.copy_(state[0])
    model.pos.copy_(state[1])
    torch.cuda.synchronize(dev)
    if model.world > 1:
        import torch.distributed as dist

        dist.barrier(group=model.group)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    with torch.cuda.stream(model._stream):
        e0.record(model._stream)
        for _ in range(new_tokens):
            model.graph.replay()
        e1.record(model._stream)
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    ms = e0.elapsed_time(e1)
    return {"tokens_per_s": model.batch * new_tokens / (ms * 1e-3), "ms_per_step": ms / new_tokens, "wall_ms_per_step": 1e3 * wall / new_tokens,
            "batch": model.batch, "prompt_len": prompt_len, "new_tokens": new_tokens}

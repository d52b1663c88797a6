"""Fused GEMV + all-gather for column-parallel layers: buffers, flags and launch helpers.

With `sal_lutgemv_grouped_exchange` the kernel that finishes an output element also stores it into
every peer GPU's gather buffer (peer-to-peer stores over NVLink) and bumps a per-launch counter on
every rank; `sal_exchange_wait` is the consumer-side wait.  This replaces "GEMV, then NCCL
all-gather" (shard.gather_columns) by one kernel plus a one-thread wait.

`PeerExchange.symmetric` allocates the buffers with torch's symmetric memory (one process per
GPU); `PeerExchange.emulated` puts all "ranks" on one GPU for tests: the ranks' launches are then
issued one after the other on one stream and every wait comes after all producers, so nothing
ever waits for a kernel that has not been launched.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch

from . import _lib, lutgemm


class PeerExchange:
    def __init__(self, world: int, rank: int, buffers: Sequence[torch.Tensor], flags: Sequence[torch.Tensor], local: int,
                 keepalive=None):
        if not 2 <= world <= _lib.SAL_MAX_PEERS:
            raise ValueError(f"world size must be 2..{_lib.SAL_MAX_PEERS}")
        self.world, self.rank = world, rank
        self.buffer = buffers[local]          # this rank's gather buffer (fp16)
        self.flags = flags[local]             # this rank's counters (int32, zero-initialised)
        self._buffer_ptrs = [int(b) if isinstance(b, int) else b.data_ptr() for b in buffers]
        self._flag_ptrs = [int(f) if isinstance(f, int) else f.data_ptr() for f in flags]
        self._keepalive = (buffers, flags, keepalive)

    # ---- constructors -------------------------------------------------------------------
    @classmethod
    def symmetric(cls, numel: int, nslots: int, group=None) -> "PeerExchange":
        """One process per GPU: buffers every rank can store into, via torch symmetric memory."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        group = group or dist.group.WORLD
        dev = torch.device("cuda", torch.cuda.current_device())
        buf = symm.empty(numel, dtype=torch.float16, device=dev)
        flg = symm.empty(nslots, dtype=torch.int32, device=dev)
        buf.zero_()
        flg.zero_()
        hb = symm.rendezvous(buf, group)
        hf = symm.rendezvous(flg, group)
        torch.cuda.synchronize(dev)
        dist.barrier(group)
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        bufs: List = [int(p) for p in hb.buffer_ptrs]
        flgs: List = [int(p) for p in hf.buffer_ptrs]
        bufs[rank], flgs[rank] = buf, flg
        return cls(world, rank, bufs, flgs, rank, keepalive=(hb, hf))

    @classmethod
    def emulated(cls, world: int, numel: int, nslots: int, device="cuda") -> List["PeerExchange"]:
        """All ranks on one GPU (tests): returns one exchange object per emulated rank."""
        bufs = [torch.zeros(numel, dtype=torch.float16, device=device) for _ in range(world)]
        flgs = [torch.zeros(nslots, dtype=torch.int32, device=device) for _ in range(world)]
        return [cls(world, r, bufs, flgs, r) for r in range(world)]

    # ---- launches -----------------------------------------------------------------------
    def _descriptor(self, gather_offsets: Sequence[int], slot: int):
        offs = (ctypes.c_longlong * len(gather_offsets))(*[int(o) for o in gather_offsets])
        ex = _lib.SalExchange()
        ex.world, ex.rank, ex.slot = self.world, self.rank, int(slot)
        for t in range(self.world):
            ex.peer_buffers[t] = self._buffer_ptrs[t]
            ex.peer_flags[t] = self._flag_ptrs[t]
        ex.gather_offsets = offs
        return ex, offs

    def prepare(self, problems, gather_offsets: Sequence[int], *, pdl: bool = False) -> "lutgemm.GroupedLaunch":
        """Grouped mode-A launch with the fused exchange, prepared once (arguments marshalled, work split
        planned, descriptors encoded).  `problems` as for lutgemm.lutgemv_grouped (mSize = LOCAL width);
        `gather_offsets[i]` = element offset of problem i's [world][mSize] block in the gather buffers.
        Call the result with the counter slot of the launch; `.writers` = this rank's arrivals per launch."""
        return lutgemm.GroupedLaunch(problems, pdl=pdl, exchange=self._descriptor(gather_offsets, 0))

    def launch(self, problems, gather_offsets: Sequence[int], slot: int, *, pdl: bool = False) -> int:
        """One-off form of `prepare` + call.  Returns this rank's arrivals."""
        prepared = self.prepare(problems, gather_offsets, pdl=pdl)
        prepared(int(slot))
        return prepared.writers

    def wait(self, slot: int, writers_per_rank: int):
        """Enqueues the wait for all ranks' arrivals on counter `slot` (and its reset)."""
        lib = _lib.load()
        dev = self.flags.device
        with torch.cuda.device(dev):
            ws = lutgemm.workspace_for(dev, 1, 8)
            _lib.check(lib.sal_exchange_wait(self.flags.data_ptr(), int(slot), self.world * int(writers_per_rank),
                                             ws.data_ptr(), torch.cuda.current_stream(dev).cuda_stream), "sal_exchange_wait")

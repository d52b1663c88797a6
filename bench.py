#!/usr/bin/env python3
"""Benchmark of the BCQ LUT-GEMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--legs a,b,...]

Headline workload (N = 1 and N > 1 alike): the LLaMA-2-7B decode linear set at batch M = 1 —
32 decoder blocks x {q,k,v,o 4096x4096; gate,up 4096x11008; down 11008x4096}, BCQ 3 bit,
group 128, power-of-two fp16 alpha, no bias, seeded synthetic tensors (no checkpoints or
datasets are available offline).  One step = one pass over all 224 products.  The products of
this workload are independent (every one has its own synthetic activation vector), so the
headline arm issues one grouped launch per decoder block (7 products, 32 launches per step),
chained with programmatic dependent launch.  The same step issued the way a decoder's data
dependencies would force it (per block: grouped q/k/v, then o, then grouped gate/up, then
down = 128 launches) is timed as well and reported under "dependency_ordered".
The 2.7 GB of weights per step exceed the 126 MB L2, so no flush is needed between steps.

Prints ONE JSON line (rank 0).  `value` = algorithmic bytes per second with everything
resident in HBM (CUDA-graph replay, CUDA events); `e2e` = the same through the Python API a
user calls, with the activations coming from pinned host memory and the results copied back,
inside the timed region.  `verify` = what the timed launches computed, compared after the timed
region with a plain fp32 torch dequantise-and-matmul on sampled output columns.  Further legs
(each a sub-record of the same line; `--legs` selects):
  overlapped_launches  the headline launches issued alternately on two streams (informational)
  cta_timeline   (not in the default set; needs the measurement build of the library) per-CTA cycle counters of
               the headline launch: dependency wait, main loop, table builds, waiting for ring data
  small_batch  the same 7B shapes with per-layer bit widths drawn from {2,3,4} (p = 0.3/0.5/0.2)
               at M in {1,4,8,16,64}: the small-batch variant of the kernel
  block_int8   the 7B shapes in the layout of the published "Lat." checkpoints (one int8 power-of-two
               multiplier triple per 8 inputs x 16 outputs), the call LutLinear.forward makes
  config5      the LLaMA-2-70B set (2 bit, GQA) at this number of GPUs, column-parallel
  decode       tokens/s of a whole decoder of the workload's architecture
  shapes       single products per shape (launches chained with PDL over a rotation of weights > L2)
`--impl reference` times the reference's CPU path (dequantise, then fp32 matmul) on this host's
cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

WORKLOADS = {
    # name: (decoder blocks, wbits, per-block launch groups of (name, K, N))
    "llama2-7b": (32, 3, ((("q_proj", 4096, 4096), ("k_proj", 4096, 4096), ("v_proj", 4096, 4096)),
                          (("o_proj", 4096, 4096),),
                          (("gate_proj", 4096, 11008), ("up_proj", 4096, 11008)),
                          (("down_proj", 11008, 4096),))),
    # the configuration the column-parallel scheme is meant for (2-bit, GQA)
    "llama2-70b": (80, 2, ((("q_proj", 8192, 8192), ("k_proj", 8192, 1024), ("v_proj", 8192, 1024)),
                           (("o_proj", 8192, 8192),),
                           (("gate_proj", 8192, 28672), ("up_proj", 8192, 28672)),
                           (("down_proj", 28672, 8192),))),
}
G = 128
BLOCK_GS = 16          # columns per multiplier of the block ("Lat." g128) layout: groupsize / 8
HEADLINE_GROUPS = [[0, 1, 2, 3, 4, 5, 6]]
DEPENDENCY_GROUPS = [[0, 1, 2], [3], [4, 5], [6]]
ALL_LEGS = ("verify", "e2e", "overlapped_launches", "dependency_ordered", "small_batch", "block_int8", "config5", "decode", "cpu_baseline",
            "reference_gpu_kernel")


def metric_name(workload, q):
    if workload == "llama2-7b":
        return "BCQ LUT-GEMV HBM GB/s, LLaMA-2-7B 3-bit g128 decode linear set, M=1"
    return f"BCQ LUT-GEMV HBM GB/s, {workload} {q}-bit g128 decode linear set, M=1"


def algorithmic_bytes(k, n, q, g=G, m=1, alpha_bytes=2):
    """Packed planes + alpha + activations (output excluded, no bias in these workloads).  The block layout has
    the same count of multipliers (one per 8 inputs x g/8 outputs), `alpha_bytes` each."""
    return k * n * q // 8 + (k // g) * n * q * alpha_bytes + 2 * m * k


def measured_peak():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons of one GPU while the timed region runs.

    Read-only NVML queries from a thread of this process every 2 ms (the timed region of a short run is a few
    tens of milliseconds: too short for `nvidia-smi -lms`, whose first line alone takes longer); `nvidia-smi` in
    a child process is the fallback where the NVML binding cannot be loaded.  `mark_begin` / `mark_end` bracket
    the timed region on the host clock; the summary uses the samples in between and says so (or, if there are
    none, all samples since the sampler was started right before the warm-up steps of the same loop)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.thread = index, [], None, None   # rows: (host time, sm MHz, max MHz, reasons)
        self.t0 = self.t1 = None
        self._stop = threading.Event()
        self.source = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:  # noqa: BLE001 - no uuid property, or not known to NVML under that name
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def __enter__(self):
        try:
            nv, handle = self._nvml_handle()
            mx = nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)
            bits = ((nv.nvmlClocksEventReasonHwSlowdown, "hw_slowdown"), (nv.nvmlClocksEventReasonHwThermalSlowdown, "hw_thermal_slowdown"),
                    (nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_thermal_slowdown"), (nv.nvmlClocksEventReasonSwPowerCap, "sw_power_cap"))

            def poll():
                while not self._stop.is_set():
                    try:
                        sm = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                        mask = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        self.rows.append((time.perf_counter(), int(sm), int(mx), [n for b, n in bits if mask & b]))
                    except Exception:  # noqa: BLE001 - a failed query is a missing sample
                        pass
                    time.sleep(0.002)

            self.source = "nvml"
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return self
        except Exception:  # noqa: BLE001 - binding or library missing: nvidia-smi below
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            c = [v.strip() for v in line.split(",")]
            if len(c) >= 6 and c[0].isdigit() and c[1].isdigit():
                self.rows.append((time.perf_counter(), int(c[0]), int(c[1]), [n for n, v in zip(self.NAMES, c[2:6]) if v.startswith("Active")]))

    def mark_begin(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.proc.wait()
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=1.0)

    def summary(self):
        rows, window = list(self.rows), "warm-up and timed steps"
        if self.t0 is not None and self.t1 is not None:
            inside = [r for r in rows if self.t0 <= r[0] <= self.t1]
            if inside:
                rows, window = inside, "timed steps"
        sm = [r[1] for r in rows]
        reasons = [n for n in self.NAMES if any(n in r[3] for r in rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(r[2] for r in rows) if rows else None,
                "reasons": reasons, "samples": len(sm), "window": window, "source": self.source}


# ------------------------------------------------------------------------------------------
# the linear set of a workload on one rank: weights, activations, outputs, launches
# ------------------------------------------------------------------------------------------
def mixed_bits(count, seed=0):
    """Per-linear bit widths of the mixed-precision configuration: {2,3,4} with p = {0.3,0.5,0.2}."""
    g = torch.Generator().manual_seed(1000003 * seed + 99)
    idx = torch.multinomial(torch.tensor([0.3, 0.5, 0.2]), count, replacement=True, generator=g)
    return [int(2 + i) for i in idx]


class LinearSet:
    """Weights of `layers` decoder blocks of a workload (column shard `rank` of `world`), drawn on the device
    from a seeded generator — packed words uniform in int32 (every bit i.i.d. +-1), alpha = 2**-k, k in
    2..8 — plus one activation vector [m, K] per product and the output slices.

    layout "row": alpha fp16 [K/128][q][N] (the configuration the metric is quoted on);
    layout "block_int8": alpha int8 [K/8][q][N/16][3], three power-of-two exponents per multiplier
    (-128 = no term), the layout LutLinear.forward hands to the kernel for a "Lat." checkpoint."""

    def __init__(self, workload, device, rank=0, world=1, *, layers=None, m=1, bits=None, seed=0, layout="row"):
        n_layers, q_default, self.groups = WORKLOADS[workload]
        self.workload, self.device, self.rank, self.world, self.m, self.layout = workload, device, rank, world, m, layout
        self.layers = n_layers if layers is None else layers
        self.per_block = sum(len(g) for g in self.groups)
        if bits is None:
            bits = [q_default] * (self.layers * self.per_block)
        self.bits = bits
        gen = torch.Generator(device=device).manual_seed(1000003 * seed + 17)
        self.blocks = []
        for li in range(self.layers):
            flat = []
            for gi, grp in enumerate(self.groups):
                for _, k, n in grp:
                    q = bits[li * self.per_block + len(flat)]
                    n_loc = n // world
                    bw = torch.randint(-2 ** 31, 2 ** 31, (k // 32, q, n_loc), dtype=torch.int32, device=device, generator=gen)
                    if layout == "row":
                        alpha = torch.exp2(-torch.randint(2, 9, (k // G, q, n_loc), device=device, generator=gen).float()).half()
                    else:
                        alpha = torch.randint(-8, -1, (k // 8, q, n_loc // BLOCK_GS, 3), device=device, generator=gen).to(torch.int8)
                        alpha[:, :, :, 2] = -128     # two terms per multiplier, the third marked absent
                    flat.append({"K": k, "N": n, "N_loc": n_loc, "q": q, "bw": bw, "alpha": alpha, "group": gi})
            self.blocks.append(flat)
        gen_x = torch.Generator(device=device).manual_seed(4242 + seed)
        n_in = sum(p["K"] for flat in self.blocks for p in flat)
        n_out = sum(p["N_loc"] for flat in self.blocks for p in flat)
        self.x_all = torch.randn(m * n_in, device=device, generator=gen_x).half()
        self.y_all = torch.zeros(m * n_out, dtype=torch.float16, device=device)
        xi = yi = 0
        for flat in self.blocks:
            for p in flat:
                p["x"] = self.x_all[xi:xi + m * p["K"]].view(m, p["K"])
                p["y"] = self.y_all[yi:yi + m * p["N_loc"]].view(m, p["N_loc"])
                p["y_off"] = yi
                xi += m * p["K"]
                yi += m * p["N_loc"]
        self.n_out_full = sum(p["N"] for flat in self.blocks for p in flat)

    def bytes_per_step(self):
        ab = 2 if self.layout == "row" else 3
        return sum(algorithmic_bytes(p["K"], p["N"], p["q"], m=self.m, alpha_bytes=ab) for flat in self.blocks for p in flat)

    def problem(self, p, fixed_acc=False):
        return dict(output=p["y_acc"] if fixed_acc else p["y"], bWeight=p["bw"], alpha=p["alpha"], bias=None, d_input=p["x"],
                    mSize=p["N_loc"], kSize=p["K"], nb=p["q"], num_groups=p["K"] // G)

    def launch_lists(self, per_block_groups, fixed_acc=False):
        """Lists of problem dicts sharing one launch: `per_block_groups` = index lists (0..6 within a block)."""
        return [[self.problem(flat[i], fixed_acc) for i in idxs] for flat in self.blocks for idxs in per_block_groups]

    def enable_accumulators(self):
        """Fixed-point accumulator outputs (int64, units of 2**-32) beside the fp16 ones, for SAL_OUT_FIXED_ATOMIC launches."""
        if hasattr(self, "y_acc_all"):
            return
        self.y_acc_all = torch.zeros(self.y_all.numel(), dtype=torch.int64, device=self.device)
        for flat in self.blocks:
            for p in flat:
                p["y_acc"] = self.y_acc_all[p["y_off"]:p["y_off"] + self.m * p["N_loc"]].view(self.m, p["N_loc"])

    def products(self, per_block_groups):
        return [[flat[i] for i in idxs] for flat in self.blocks for idxs in per_block_groups]


def torch_reference_columns(p, cols, m_rows=None):
    """fp32 dequantise-then-matmul of product `p` on output columns `cols` (a plain torch restatement of
    y = x @ W.T with W = sum_b alpha_b * sign_b; the oracle of the test-suite is the authority, this is the
    benchmark's own after-the-fact check of what it timed)."""
    bw, k = p["bw"][:, :, cols], p["K"]
    shifts = torch.arange(32, device=bw.device, dtype=torch.int32).view(1, 32, 1, 1)
    sign = (((bw.unsqueeze(1) >> shifts) & 1).float() * 2 - 1).reshape(k, bw.shape[1], len(cols))      # [K, q, C]
    if p["alpha"].dtype == torch.float16:
        a = p["alpha"][:, :, cols].float().repeat_interleave(G, dim=0)                                  # [K, q, C]
    else:
        e = p["alpha"].float()
        mult = torch.where(e == -128, torch.zeros_like(e), torch.exp2(e)).sum(-1)                      # [K/8, q, N/16]
        a = mult[:, :, cols // BLOCK_GS].repeat_interleave(8, dim=0)
    w = (sign * a).sum(1)                                                                               # [K, C]
    x = p["x"] if m_rows is None else p["x"][:m_rows]
    return x.float() @ w


def sample_columns(n, count=384, seed=0):
    """Output columns to check: both sides of every 256-column tile boundary (the kernel's column ranges
    are whole tiles), the first and last columns, and a seeded random sample."""
    cols = {0, 1, n - 2, n - 1}
    for t in range(256, n, 256):
        cols.update((t - 1, t))
    g = torch.Generator().manual_seed(seed + n)
    cols.update(int(c) for c in torch.randint(0, n, (count,), generator=g))
    return sorted(c for c in cols if 0 <= c < n)


def verify_products(products, device, fixed_acc=False):
    """Max relative error (max|y - ref| / max|ref| per product) of outputs already computed, over sampled columns."""
    worst = 0.0
    for p in products:
        cols = torch.tensor(sample_columns(p["N_loc"]), device=device)
        ref = torch_reference_columns(p, cols)
        got = (p["y_acc"][:, cols].double() / float(2 ** 32)).float() if fixed_acc else p["y"][:, cols].float()
        worst = max(worst, float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)))
    return worst


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
class Timer:
    def __init__(self, args, device, world, stream):
        self.args, self.device, self.world, self.stream = args, device, world, stream

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize(self.device)

    def capture(self, one_step):
        with torch.cuda.stream(self.stream):
            one_step()                       # also sizes the workspace and runs the one-off probes
            torch.cuda.synchronize(self.device)
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    one_step()
                return g.replay, True
            except Exception as exc:  # noqa: BLE001 - a failed capture (e.g. of a collective) falls back to eager launches
                print(f"[bench] graph capture failed ({type(exc).__name__}: {exc}); timing eager launches", file=sys.stderr)
                torch.cuda.synchronize(self.device)
                return one_step, False

    def timed(self, fn, steps, warmup=None, clocks=False):
        """ms per step: CUDA events on the launch stream around `steps` calls, max over ranks."""
        with torch.cuda.stream(self.stream):
            clk = ClockSampler(self.device.index) if clocks else None
            if clk:
                clk.__enter__()     # already running during the warm-up steps: no start-up gap at the timed ones
            for _ in range(max(self.args.warmup if warmup is None else warmup, 3)):
                fn()
            self.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if clk:
                clk.mark_begin()
            e0.record(self.stream)
            for _ in range(steps):
                fn()
            e1.record(self.stream)
            self.barrier()
            if clk:
                clk.mark_end()
                clk.__exit__()
            ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], dtype=torch.float64, device=self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps, clk


class SetRunner:
    """The launches of a LinearSet in one arrangement, on one GPU or column-parallel with the output slices
    gathered either inside the kernel (peer stores + counters) or by NCCL."""

    def __init__(self, lset, per_block_groups, *, peer=None, y_full=None, nslots=4, fixed_acc=False):
        from shiftaddllm_b200 import lutgemm

        self.lset, self.peer, self.y_full, self.nslots = lset, peer, y_full, nslots
        self.products = lset.products(per_block_groups)
        if fixed_acc:     # one GPU only: outputs are fixed-point accumulators the products add into (no split-K reduction tail)
            lset.enable_accumulators()
            self.sequence = None
            self.prepared = [lutgemm.prepare_grouped(plist, pdl=True, atomic_fixed=True) for plist in lset.launch_lists(per_block_groups, True)]
            return
        self.sequence = None
        self.gather_slices = []          # NCCL: (gathered view, local view) per launch
        self.gather_offsets = []         # fused: per launch, per product, element offset of its [world][N_loc] block
        world = lset.world
        self.prepared = []
        yfi = 0
        for prods, plist in zip(self.products, lset.launch_lists(per_block_groups)):
            if world == 1:
                self.prepared.append(lutgemm.prepare_grouped(plist, pdl=True))
                continue
            if peer is not None:
                offs = []
                for p in prods:
                    offs.append(yfi)
                    yfi += p["N"]
                self.gather_offsets.append(offs)
                self.prepared.append(peer.prepare(plist, offs, pdl=True))
            else:
                lo, hi = prods[0]["y_off"], prods[-1]["y_off"] + prods[-1]["N_loc"]
                self.gather_slices.append((y_full[yfi:yfi + (hi - lo) * world], lset.y_all[lo:hi]))
                yfi += (hi - lo) * world
                self.prepared.append(lutgemm.prepare_grouped(plist, pdl=True))

    def step(self):
        if self.lset.world == 1:
            if self.sequence is None:       # the whole step enqueued by one call into the library
                from shiftaddllm_b200 import lutgemm

                self.sequence = lutgemm.LaunchSequence(self.prepared)
            self.sequence()
        elif self.peer is not None:
            for li, launch in enumerate(self.prepared):
                slot = li % self.nslots
                launch(slot)
                self.peer.wait(slot, launch.writers)
        else:
            import torch.distributed as dist

            for launch, (full, local) in zip(self.prepared, self.gather_slices):
                launch()
                dist.all_gather_into_tensor(full, local)

    def step_two_streams(self, side):
        """The same launches with the even ones on the current stream and the odd ones on `side` (one GPU; the
        products of different launches are independent, each stream has its own scratch buffer): a launch no longer
        waits for the last thread block of the launch in front of it, only for the one before that."""
        from shiftaddllm_b200 import lutgemm

        if getattr(self, "_split", None) is None:
            self._split = (lutgemm.LaunchSequence(self.prepared[0::2]), lutgemm.LaunchSequence(self.prepared[1::2]))
        cur = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(cur)
        side.wait_event(fork)
        with torch.cuda.stream(side):
            self._split[1]()
            join = torch.cuda.Event()
            join.record(side)
        self._split[0]()
        cur.wait_event(join)

    def exchange_check(self):
        """After a step: the gather buffer of every launch against an NCCL all-gather of the local slices."""
        import torch.distributed as dist

        lset, world = self.lset, self.lset.world
        gathered = [torch.empty_like(lset.y_all) for _ in range(world)]
        dist.all_gather(gathered, lset.y_all)
        src = self.peer.buffer if self.peer is not None else self.y_full
        bad = 0
        if self.peer is not None:
            for prods, offs in zip(self.products, self.gather_offsets):
                for p, off in zip(prods, offs):
                    for r in range(world):
                        want = gathered[r][p["y_off"]:p["y_off"] + p["N_loc"]]
                        got = src[off + r * p["N_loc"]: off + (r + 1) * p["N_loc"]]
                        bad += int(not torch.equal(want, got))
        else:
            for prods, (full, local) in zip(self.products, self.gather_slices):
                lo, hi = prods[0]["y_off"], prods[-1]["y_off"] + prods[-1]["N_loc"]
                for r in range(world):
                    bad += int(not torch.equal(full[r * (hi - lo):(r + 1) * (hi - lo)], gathered[r][lo:hi]))
        t = torch.tensor([bad], device=lset.device)
        dist.all_reduce(t)
        return "bit-identical" if int(t.item()) == 0 else f"{int(t.item())} slices differ"


def make_peer(args, world, device, numel):
    """Peer buffers for the fused exchange, or None (every rank then takes the NCCL path)."""
    import torch.distributed as dist

    if world == 1 or args.exchange != "fused":
        return None
    from shiftaddllm_b200.exchange import PeerExchange

    peer = None
    try:
        peer = PeerExchange.symmetric(numel, nslots=4)
        ok = torch.ones(1, device=device)
    except Exception as exc:  # noqa: BLE001 - no peer-mappable memory on this box: use NCCL on every rank
        print(f"[bench] symmetric memory unavailable ({type(exc).__name__}: {exc}); using the NCCL exchange", file=sys.stderr)
        ok = torch.zeros(1, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)   # all ranks take the same path
    return peer if bool(ok.item()) else None


def device_status(lib, device, stream):
    from shiftaddllm_b200 import lutgemm

    with torch.cuda.stream(stream):   # the workspace is cached per (device, stream)
        ws = lutgemm.workspace_for(device, 1, 8)
    return lib.sal_workspace_status(ws.data_ptr(), stream.cuda_stream)


def run_ours(args, rank, world, device):
    from shiftaddllm_b200 import _lib

    lib = _lib.load()
    _lib.check(lib.sal_device_ok(), "sal_device_ok")
    legs = set(args.legs)
    n_layers, q, _ = WORKLOADS[args.workload]
    stream = torch.cuda.Stream(device)
    timer = Timer(args, device, world, stream)

    lset = LinearSet(args.workload, device, rank, world, layers=args.layers)
    n_layers = lset.layers
    peer = make_peer(args, world, device, lset.n_out_full)
    fused = peer is not None
    y_full = torch.zeros(lset.n_out_full, dtype=torch.float16, device=device) if (world > 1 and not fused) else None
    head = SetRunner(lset, HEADLINE_GROUPS, peer=peer, y_full=y_full)
    replay, graphed = timer.capture(head.step)
    ms_per_step, clk = timer.timed(replay, args.steps, clocks=True)
    total = lset.bytes_per_step()
    peak, which = measured_peak()
    n_launch = len(head.prepared)
    per_launch_us = ms_per_step * 1e3 / n_launch
    achieved = total / world / (ms_per_step * 1e-3) / 1e9   # per GPU: this rank's bytes over the step time

    out = {
        "metric": metric_name(args.workload, q), "value": round(total / (ms_per_step * 1e-3) / 1e9, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 in, fp32 accumulate",
        "data": "synthetic", "impl": "ours",
        "config": {"workload": f"{args.workload} decode linear set ({n_layers} blocks x 7 linears), M=1, BCQ {q}-bit g128",
                   "launches_per_step": n_launch,
                   "launch_structure": ("one grouped launch per decoder block (7 independent products); PDL chained; "
                                        + ("CUDA graph" if graphed else "eager")),
                   "l2": f"inputs larger than L2 ({total / 1e9:.1f} GB of weights per step), no flush",
                   "parallelism": (f"column-parallel x{world}, all-gather "
                                   + ("fused into the kernel (peer-to-peer stores + counters)" if fused else "by NCCL"))
                   if world > 1 else "single GPU"},
        "tokens_per_s_linears_only": round(1e3 / ms_per_step, 1),
        "gemv_per_s": round(n_layers * 7 * 1e3 / ms_per_step, 1),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "peak_source": f"{which} copy bandwidth (MEASURED_PEAKS.json)" if which == "measured" else "fallback 6650",
                     "kernel": f"lutgemv_tiled_kernel<{q},8>", "avg_launch_us": round(per_launch_us, 3),
                     "algorithmic_bytes_per_launch": total // world // n_launch,
                     "traffic": read_traffic() if (args.workload == "llama2-7b" and world == 1) else None},
        "gpu_launches": n_launch * args.steps,
        "clocks": clk.summary(),
    }

    # ---- what the timed launches computed (after the timed region): block 0 and the last block
    if "verify" in legs:
        with torch.cuda.stream(stream):
            lset.y_all.zero_()
            replay()
            torch.cuda.synchronize(device)
            check = [p for prods in (head.products[0], head.products[-1]) for p in prods]
            out["verify"] = {"max_rel_err": round(verify_products(check, device), 6), "tolerance": 1e-2,
                             "checked": "all 7 products of the first and the last decoder block of the timed headline launches, "
                                        "sampled output columns (tile boundaries + random)",
                             "checker": "fp32 torch dequantise + matmul on the same device tensors"}
            if world > 1:
                out["exchange_check"] = head.exchange_check()

    # ---- the same launches issued alternately on two streams (informational: shows what the wait for the last thread
    # block of the launch in front costs a chain of launches)
    if "overlapped_launches" in legs and world == 1:
        side = torch.cuda.Stream(device)
        two_replay, two_graphed = timer.capture(lambda: head.step_two_streams(side))
        two_ms, _ = timer.timed(two_replay, args.steps)
        rec = {"ms_per_step": round(two_ms, 4), "value": round(total / (two_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
               "frac_of_measured_hbm": round(total / (two_ms * 1e-3) / 1e9 / peak, 4),
               "structure": "the headline launches, even ones on one stream and odd ones on a second (each PDL chained, own "
                            "scratch buffer), " + ("one CUDA graph" if two_graphed else "eager")}
        if "verify" in legs:
            with torch.cuda.stream(stream):
                lset.y_all.zero_()
                two_replay()
                torch.cuda.synchronize(device)
                rec["verify_max_rel_err"] = round(verify_products([p for prods in (head.products[0], head.products[1], head.products[-1])
                                                                   for p in prods], device), 6)
        out["overlapped_launches"] = rec

    # ---- per-CTA cycle counters of the headline launches (measurement build of the library only)
    if "cta_timeline" in legs and world == 1:
        out["cta_timeline"] = cta_timeline_record(lib, replay, device, clk.summary().get("sm_mhz") or 1965)

    # ---- the same step in the order a decoder's data dependencies force
    dep = None
    if "dependency_ordered" in legs:
        dep = SetRunner(lset, DEPENDENCY_GROUPS, peer=peer, y_full=y_full)
        dep_replay, _ = timer.capture(dep.step)
        dep_ms, _ = timer.timed(dep_replay, max(3, args.steps // 4))
        rec = {"launches_per_step": len(dep.prepared), "ms_per_step": round(dep_ms, 4),
               "value": round(total / (dep_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
               "structure": "per block: grouped{q,k,v}, o, grouped{gate,up}, down; PDL chained"}
        if "verify" in legs:
            with torch.cuda.stream(stream):
                lset.y_all.zero_()
                dep_replay()
                torch.cuda.synchronize(device)
                rec["verify_max_rel_err"] = round(verify_products([p for prods in dep.products[:4] for p in prods], device), 6)
                if world > 1:
                    rec["exchange_check"] = dep.exchange_check()
        out["dependency_ordered"] = rec
        if world == 1:
            # the same launches with fixed-point accumulator outputs (int64, integer atomics: no reduction tail on the
            # critical path of a dependent launch, still bit-identical from run to run) — what the decoder issues
            acc = SetRunner(lset, DEPENDENCY_GROUPS, fixed_acc=True)
            acc_replay, _ = timer.capture(acc.step)
            acc_ms, _ = timer.timed(acc_replay, max(3, args.steps // 4))
            rec = {"launches_per_step": len(acc.prepared), "ms_per_step": round(acc_ms, 4), "value": round(total / (acc_ms * 1e-3) / 1e9, 1),
                   "unit": "GB/s", "structure": "as dependency_ordered, outputs added into 64-bit fixed-point accumulators"}
            if "verify" in legs:
                with torch.cuda.stream(stream):
                    lset.y_acc_all.zero_()
                    acc_replay()
                    torch.cuda.synchronize(device)
                    rec["verify_max_rel_err"] = float(f"{verify_products([p for prods in acc.products[:4] for p in prods], device, True):.3g}")
                    first = lset.y_acc_all.clone()
                    lset.y_acc_all.zero_()
                    acc_replay()
                    torch.cuda.synchronize(device)
                    rec["bit_identical_repeat"] = bool(torch.equal(first, lset.y_acc_all))
            out["dependency_ordered_fixed_accumulators"] = rec
            del acc, acc_replay

    # ---- end to end: host activations in, host results out, through the public Python API
    if "e2e" in legs:
        # Host buffers in, host buffers out, every step.  The PCIe copies run on two further streams into / out of
        # device staging buffers, so that they overlap the neighbouring steps' kernels; the compute stream only
        # does two device-to-device copies per step (activations in, results out).
        x_host = lset.x_all.cpu().pin_memory()
        y_src = (peer.buffer if fused else y_full) if world > 1 else lset.y_all
        y_host = torch.empty(y_src.shape, dtype=torch.float16).pin_memory()
        x_stage, y_stage = torch.empty_like(lset.x_all), torch.empty_like(y_src)
        in_stream, out_stream = torch.cuda.Stream(device), torch.cuda.Stream(device)   # one PCIe direction each
        e2e_steps = max(3, min(args.steps, 10))
        ev_x_in = [torch.cuda.Event() for _ in range(e2e_steps + 2)]      # activations of step i are on the device
        ev_x_used = [torch.cuda.Event() for _ in range(e2e_steps + 2)]    # step i has taken them out of the staging buffer
        ev_y_out = [torch.cuda.Event() for _ in range(e2e_steps + 2)]     # results of step i are in the staging buffer
        ev_y_done = [torch.cuda.Event() for _ in range(e2e_steps + 2)]    # ... and have left for the host

        def e2e_step(i):
            with torch.cuda.stream(in_stream):
                if i > 0:
                    in_stream.wait_event(ev_x_used[i - 1])
                x_stage.copy_(x_host, non_blocking=True)
                ev_x_in[i].record(in_stream)
            stream.wait_event(ev_x_in[i])
            lset.x_all.copy_(x_stage, non_blocking=True)
            ev_x_used[i].record(stream)
            replay()
            if i > 0:
                stream.wait_event(ev_y_done[i - 1])
            y_stage.copy_(y_src, non_blocking=True)
            ev_y_out[i].record(stream)
            with torch.cuda.stream(out_stream):
                out_stream.wait_event(ev_y_out[i])
                y_host.copy_(y_stage, non_blocking=True)
                ev_y_done[i].record(out_stream)

        with torch.cuda.stream(stream):
            e2e_step(0)
            timer.barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                e2e_step(i + 1)
            torch.cuda.synchronize(device)          # every step's results have reached the host buffer
            timer.barrier()
            e2e_s = (time.perf_counter() - t0) / e2e_steps
        t = torch.tensor([e2e_s], dtype=torch.float64, device=device)
        if world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
        out["e2e"] = {"value": round(total / e2e_s / 1e9, 1), "unit": "GB/s", "ms_per_step": round(e2e_s * 1e3, 3),
                      "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                      "api": ("shiftaddllm_b200.lutgemm.prepare_grouped launches (prepared once, enqueued through lutgemm.LaunchSequence), "
                              + ("the step's launches replayed as a CUDA graph" if graphed else "enqueued eagerly") + "; every step copies its activations in from pinned host memory and its results out "
                              "to pinned host memory, the PCIe copies on two further streams (one per direction) overlapping the neighbouring steps")}
        del x_stage, y_stage
    out["device_status"] = device_status(lib, device, stream)

    del head, dep, replay
    if world > 1 and "config5" in legs and args.workload == "llama2-7b":
        del lset
        torch.cuda.empty_cache()
        out["config5"] = config5_record(args, timer, rank, world, device, peer_factory=lambda n: make_peer(args, world, device, n))
        return out if rank == 0 else None
    if rank != 0:
        return None
    if world == 1:
        if "small_batch" in legs and args.workload == "llama2-7b":
            out["small_batch"] = small_batch_record(args, timer, device)
        if "block_int8" in legs and args.workload == "llama2-7b":
            out["block_int8"] = block_layout_record(args, timer, device)
        del lset
        torch.cuda.empty_cache()
        if "config5" in legs and args.workload == "llama2-7b":
            out["config5"] = config5_record(args, timer, rank, world, device, peer_factory=None)
        if "cpu_baseline" in legs:
            out["cpu_baseline"] = cpu_reference(args.workload, sample_layers=1, reps=5)
        if "reference_gpu_kernel" in legs:
            out["reference_gpu_kernel"] = reference_gpu_kernel()
        if "decode" in legs:
            torch.cuda.empty_cache()
            out["decode"] = decode_tokens_per_s(args.workload, device)
    return out


def config5_record(args, timer, rank, world, device, peer_factory):
    """The LLaMA-2-70B linear set (2 bit, GQA, 80 blocks) at this number of GPUs: the configuration the
    column-parallel scheme is meant for."""
    lset = LinearSet("llama2-70b", device, rank, world, seed=5)
    peer = peer_factory(lset.n_out_full) if peer_factory else None
    y_full = torch.zeros(lset.n_out_full, dtype=torch.float16, device=device) if (world > 1 and peer is None) else None
    total = lset.bytes_per_step()
    rec = {"workload": "llama2-70b decode linear set (80 blocks x 7 linears), M=1, BCQ 2-bit g128", "n_gpus": world}
    for name, groups in (("block_launches", HEADLINE_GROUPS), ("dependency_ordered", DEPENDENCY_GROUPS)):
        run = SetRunner(lset, groups, peer=peer, y_full=y_full)
        replay, _ = timer.capture(run.step)
        ms, _ = timer.timed(replay, max(3, min(args.steps, 20)))
        sub = {"ms_per_step": round(ms, 4), "value": round(total / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
               "launches_per_step": len(run.prepared), "avg_launch_us": round(ms * 1e3 / len(run.prepared), 3)}
        if "verify" in args.legs:
            with torch.cuda.stream(timer.stream):
                lset.y_all.zero_()
                replay()
                torch.cuda.synchronize(device)
                sub["verify_max_rel_err"] = round(verify_products([p for p in run.products[0]] + [p for p in run.products[-1]], device), 6)
                if world > 1:
                    sub["exchange_check"] = run.exchange_check()
        rec[name] = sub
        del run, replay
    peak, _ = measured_peak()
    rec["roofline_frac_of_measured"] = round(rec["block_launches"]["value"] / world / peak, 4)
    del lset, peer, y_full
    torch.cuda.empty_cache()
    if "decode" in args.legs:
        rec["decoder"] = sharded_decoder_record(args, rank, world, device)
    return rec


def cta_timeline_record(lib, replay, device, sm_mhz):
    """Where the thread blocks of the headline launch spend their time: the cycle counters a library built with
    -DSAL_MEASURE keeps per CTA (SAL_LUTGEMM_LIBRARY=.../libsal_lutgemm_measure.so), read after one more replay."""
    import numpy as np

    if not hasattr(lib, "sal_debug_read"):
        return {"unavailable": "the loaded library is not a measurement build (python -m shiftaddllm_b200.build --measure, "
                               "then SAL_LUTGEMM_LIBRARY=shiftaddllm_b200/libsal_lutgemm_measure.so)"}
    replay()
    torch.cuda.synchronize(device)
    buf = np.zeros(1024 * 8, dtype=np.uint64)
    if lib.sal_debug_read(buf.ctypes.data, buf.nbytes) != 0:
        return {"unavailable": "sal_debug_read failed"}
    d = buf.reshape(512, 2, 8)[:, 0, :].astype(np.float64)       # consumer warp 0 of every CTA of the last launch
    d = d[d[:, 4] > 0]
    us = lambda col: d[:, col] / sm_mhz
    rec = {"ctas": int(len(d)), "sm_mhz": sm_mhz, "units_per_cta": round(float(d[:, 4].mean()), 2),
           "k_blocks_per_cta": round(float(d[:, 5].mean()), 2),
           "dependency_wait_us": {"mean": round(float(us(0).mean()), 2), "first_ctas": round(float(us(0)[:16].mean()), 2),
                                  "last_ctas": round(float(us(0)[-16:].mean()), 2)},
           "main_loop_us": {"mean": round(float(us(3).mean()), 2), "min": round(float(us(3).min()), 2), "max": round(float(us(3).max()), 2)},
           "of_which_table_builds_us": round(float(us(2).mean()), 2), "of_which_waiting_for_ring_data_us": round(float(us(1).mean()), 2),
           "ctas_per_sm": round(len(d) / max(1, len(set(d[:, 6].astype(int)))), 2), "by_problem": []}
    for p in sorted(set(d[:, 7].astype(int))):
        m = d[:, 7].astype(int) == p
        rec["by_problem"].append({"problem": int(p), "ctas": int(m.sum()),
                                  "lookup_us_per_unit": round(float(((d[m, 3] - d[m, 2]) / d[m, 4]).mean() / sm_mhz), 3),
                                  "dependency_wait_us": round(float(us(0)[m].mean()), 2)})
    return rec


def sharded_decoder_record(args, rank, world, device):
    """tokens/s of the column-parallel decoder of the 70B architecture (80 blocks, hidden 8192, 64 query / 8 kv
    heads, FFN 28672, BCQ 2 bit) at this number of GPUs: batch 1 (all-gather fused into the GEMV kernels) and 16
    sequences in lock step (M = 16 products, NCCL all-gather), 128 new tokens after a 1024-token prompt.  Before
    that, on a small shape, the column-parallel logits are compared with a single-GPU decoder of the same seed."""
    import torch.distributed as dist

    from shiftaddllm_b200 import decoder, shard_decoder

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    rec = {"workload": "llama2-70b-shaped decoder, BCQ 2-bit g128 linears column-parallel over the GPUs, replicated attention / "
                       "norms / fp16 lm_head, 1024-token prompt of uniform random ids, 128 greedy tokens, one CUDA graph per token",
           "n_gpus": world}
    # ---- correctness on a small shape: same model (same seed) on one GPU and column-parallel
    small = decoder.LlamaShape(512, 2, 8, 8, 1024, vocab=1000)
    par = shard_decoder.ColumnParallelDecoder(small, wbits=2, max_len=32, rank=rank, world=world, device=device, seed=9,
                                              exchange=args.exchange)
    one = decoder.BcqLlamaDecoder(small, wbits=2, max_len=32, device=device, seed=9, fused=True)
    par.reset()
    one.reset()
    worst = 0.0
    for t in (5, 17, 999, 3, 42):
        par.token.fill_(t)
        one.token.fill_(t)
        par.step()
        one.step()
        torch.cuda.synchronize(device)
        worst = max(worst, float((par.logits[0] - one.logits).abs().max() / one.logits.abs().max()))
    rec["check_vs_single_gpu_decoder"] = {"max_rel_err_logits": round(max_over_ranks(worst), 6), "tolerance": 2e-2,
                                          "logits_absmax": round(float(one.logits.abs().max()), 4),
                                          "shape": "hidden 512, 2 blocks, 8 heads, 8 kv heads, FFN 1024"}
    del par, one
    torch.cuda.empty_cache()
    shape = decoder.SHAPES["llama2-70b"]
    prompt, new = 1024, 128
    for batch in (1, 16):
        model = shard_decoder.ColumnParallelDecoder(shape, wbits=2, max_len=prompt + new + 16, batch=batch, rank=rank, world=world,
                                                    device=device, seed=0, exchange=args.exchange)
        if batch == 1:
            r = shard_decoder.benchmark(model, prompt, new)
            fill = "prompt fed through the model, one step per token"
        else:
            # the cache of the prompt positions is filled with synthetic values instead of 1024 model steps per
            # sequence: the timed steps read the same number of cached positions either way
            model.capture()
            model.reset()
            gen = torch.Generator(device=device).manual_seed(11)
            model.k_cache[:, :, :prompt].copy_(0.5 * torch.randn(model.k_cache[:, :, :prompt].shape, device=device, generator=gen))
            model.v_cache[:, :, :prompt].copy_(0.5 * torch.randn(model.v_cache[:, :, :prompt].shape, device=device, generator=gen))
            model.pos.fill_(prompt)
            r = shard_decoder.benchmark_steps(model, new)
            fill = "cache of the prompt positions filled with synthetic values (same positions read per step)"
        ms = max_over_ranks(r["ms_per_step"])
        rec[f"batch{batch}"] = {"tokens_per_s": round(batch * 1e3 / ms, 1), "ms_per_step": round(ms, 4), "prompt": fill,
                                "exchange": "fused into the GEMV kernels" if model.fused else ("NCCL all-gather" if world > 1 else "none")}
        del model
        torch.cuda.empty_cache()
    if world == 1:
        # what one GPU is best at: no exchange, so the products can add into fixed-point accumulators (no split-K tail)
        model = decoder.BcqLlamaDecoder(shape, 2, G, max_len=prompt + 2 * new + 16, device=device, atomic=True)
        r = decoder.benchmark(model, prompt, new)
        rec["batch1_fixed_accumulators"] = {"tokens_per_s": round(r["tokens_per_s"], 1), "ms_per_step": round(r["ms_per_token"], 4),
                                            "prompt": "prompt fed through the model in chunks of 64 tokens",
                                            "structure": "single-GPU decoder, products add into 64-bit fixed-point accumulators"}
        del model
        torch.cuda.empty_cache()
    return rec


def small_batch_record(args, timer, device):
    """The 7B shapes with per-linear bit widths drawn from {2,3,4} and M activation rows: the half2-table
    small-batch variant.  A grouped launch with mixed widths is one kernel per distinct width."""
    n_layers, _, groups = WORKLOADS["llama2-7b"]
    bits = mixed_bits(n_layers * 7)
    rec = {"workload": "llama2-7b linear set, per-linear wbits from {2,3,4} (p = 0.3/0.5/0.2), g128; one grouped launch "
                       "per decoder block and distinct width, PDL chained, CUDA graph",
           "bits_histogram": {str(b): bits.count(b) for b in (2, 3, 4)},
           "bound_note": "M >= 8 is bound by shared-memory table lookups (M/2 lookups per weight byte), not by HBM"}
    peak, _ = measured_peak()
    for m in (1, 4, 8, 16, 64):
        lset = LinearSet("llama2-7b", device, bits=bits, m=m, seed=3)
        run = SetRunner(lset, HEADLINE_GROUPS)
        replay, _ = timer.capture(run.step)
        steps = max(3, min(args.steps, 20 if m <= 8 else 5))
        ms, _ = timer.timed(replay, steps)
        total = lset.bytes_per_step()
        sub = {"ms_per_step": round(ms, 4), "value": round(total / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
               "frac_of_measured_hbm": round(total / (ms * 1e-3) / 1e9 / peak, 4),
               "rows_per_s": round(m * 1e3 / ms, 1)}
        if "verify" in args.legs:
            with torch.cuda.stream(timer.stream):
                lset.y_all.zero_()
                replay()
                torch.cuda.synchronize(device)
                sub["verify_max_rel_err"] = round(verify_products(run.products[0], device), 6)
        rec[f"M={m}"] = sub
        del lset, run, replay
        torch.cuda.empty_cache()
    return rec


def block_layout_record(args, timer, device):
    """The 7B shapes in the block layout of the published "Lat." checkpoints (groupsize 128: one multiplier per
    8 inputs x 16 outputs, int8 power-of-two exponents): lutgemm_compute_block_shiftInt8, the call
    LutLinear.forward makes.  One launch per product, PDL chained, CUDA graph."""
    from shiftaddllm_b200 import lutgemm

    lset = LinearSet("llama2-7b", device, layout="block_int8", seed=7)
    plist = [p for flat in lset.blocks for p in flat]

    def step():
        for p in plist:
            lutgemm.lutgemm_block_fused(p["y"], p["bw"], p["alpha"], None, p["x"], p["N"], p["K"], p["q"], p["N"] // BLOCK_GS, pdl=True)

    replay, _ = timer.capture(step)
    ms, _ = timer.timed(replay, max(3, min(args.steps, 20)))
    total = lset.bytes_per_step()
    peak, _ = measured_peak()
    rec = {"workload": "llama2-7b linear set, M=1, BCQ 3-bit, block layout alpha int8 [K/8][3][N/16][3]; one launch per product",
           "launches_per_step": len(plist), "ms_per_step": round(ms, 4), "value": round(total / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
           "frac_of_measured_hbm": round(total / (ms * 1e-3) / 1e9 / peak, 4), "avg_launch_us": round(ms * 1e3 / len(plist), 3)}
    if "verify" in args.legs:
        with torch.cuda.stream(timer.stream):
            lset.y_all.zero_()
            replay()
            torch.cuda.synchronize(device)
            rec["verify_max_rel_err"] = round(verify_products(lset.blocks[0], device), 6)
    return rec


def shapes_record(args, timer, device):
    """Single products, one per launch, launches chained with PDL over a rotation of distinct weight tensors
    whose total exceeds L2: microseconds per call, GB/s of algorithmic bytes and fraction of the measured peak."""
    from shiftaddllm_b200 import lutgemm

    peak, _ = measured_peak()
    rows = []
    for spec in args.shapes.split(","):
        k, n = (int(v) for v in spec.lower().split("x"))
        for q in (int(v) for v in args.wbits.split(",")):
            for m in (int(v) for v in args.batch.split(",")):
                per = k * n * q // 8
                copies = max(4, min(64, -(-(256 << 20) // per)))
                gen = torch.Generator(device=device).manual_seed(k * 31 + n * 7 + q)
                bws = [torch.randint(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=torch.int32, device=device, generator=gen)
                       for _ in range(copies)]
                x = torch.randn(m, k, device=device, generator=gen).half()
                y = torch.empty(m, n, dtype=torch.float16, device=device)
                if args.mode == "block_int8":     # the layout of the "Lat." checkpoints: LutLinear.forward's call
                    alpha = torch.randint(-8, -1, (k // 8, q, n // BLOCK_GS, 3), device=device, generator=gen).to(torch.int8)
                    alpha[:, :, :, 2] = -128
                    launches = None

                    def step():
                        for bw in bws:
                            lutgemm.lutgemm_block_fused(y, bw, alpha, None, x, n, k, q, n // BLOCK_GS, pdl=True)
                else:
                    alpha = torch.exp2(-torch.randint(2, 9, (k // G, q, n), device=device, generator=gen).float()).half()
                    launches = [lutgemm.prepare_grouped([dict(output=y, bWeight=bw, alpha=alpha, bias=None, d_input=x, mSize=n, kSize=k,
                                                              nb=q, num_groups=k // G)], pdl=True) for bw in bws]

                    def step():
                        for launch in launches:
                            launch()

                replay, _ = timer.capture(step)
                ms, _ = timer.timed(replay, 10)
                us = ms * 1e3 / copies
                nbytes = algorithmic_bytes(k, n, q, m=m, alpha_bytes=3 if args.mode == "block_int8" else 2)
                rows.append({"K": k, "N": n, "q": q, "M": m, "mode": args.mode, "us_per_call": round(us, 3), "gbps": round(nbytes / us / 1e3, 1),
                             "frac_of_measured_hbm": round(nbytes / us / 1e3 / peak, 4)})
                del launches, bws, replay
    return rows


def decode_tokens_per_s(workload, device):
    """The other half of the metric: greedy batch-1 decode of a whole decoder of the workload's
    architecture (random init, every linear a synthetic BCQ layer): 128 new tokens after a
    512-token prompt (1024 for the 70B shape), the step replayed as one CUDA graph.  Reported for
    fixed-order fp16 GEMV outputs and for the opt-in fixed-point atomic accumulation; for the 7B shape also 16
    sequences decoded in lock step (64 new tokens each) on the small-batch kernel."""
    from shiftaddllm_b200 import decoder

    q = WORKLOADS[workload][1]
    prompt = 512 if workload == "llama2-7b" else 1024
    with torch.cuda.device(device):
        model = decoder.BcqLlamaDecoder(decoder.SHAPES[workload], q, G, max_len=prompt + 2 * 128 + 16, device=device)
        res = {}
        for name, atomic in (("fp16_outputs", False), ("fixed_atomic_outputs", True)):
            model.set_atomic(atomic)
            r = decoder.benchmark(model, prompt, 128)
            res[name] = {"tokens_per_s": round(r["tokens_per_s"], 1), "ms_per_token": round(r["ms_per_token"], 4),
                         "median_ms_per_token_synced": round(r["median_ms_per_token_synced"], 4)}
        if workload == "llama2-7b":
            # 16 sequences in lock step: the linears run the small-batch (M = 16) LUT kernel
            batch = decoder.BcqLlamaBatchDecoder(decoder.SHAPES[workload], q, G, max_len=prompt + 64 + 16, batch=16, device=device,
                                                 like=model)
            r = decoder.benchmark_batch(batch, prompt, 64)
            res["batch16_fp16_outputs"] = {"tokens_per_s": round(r["tokens_per_s"], 1), "ms_per_step": round(r["ms_per_step"], 3),
                                           "new_tokens_per_sequence": 64}
    res["workload"] = (f"{workload}-shaped decoder, BCQ {q}-bit g128 linears, fp16 lm_head, batch 1, {prompt}-token prompt of "
                       "uniform random ids, 128 greedy tokens, one CUDA graph per token")
    return res


def read_traffic():
    """Per-launch DRAM traffic (bytes) of the dominant kernel, taken from the committed ncu summary
    (dram__bytes_read.sum + dram__bytes_write.sum, mean over the launch types of a decoder block)."""
    import re

    path = os.path.join(REPO, "profiles", "lutgemv_tiled_q3_decoder_block_full.md")
    try:
        m = re.search(r"Mean traffic per launch ([0-9 ]+) B", open(path).read())
        return int(m.group(1).replace(" ", "")) if m else None
    except OSError:
        return None


def reference_gpu_kernel():
    """Informational: the reference's own CUDA kernel (mode A, M = 1; lut_gemm/mv_fp16_bias.hpp:498-579 through
    nqmv_bias_shift_mulq) timed on this GPU on the three 7B shapes by the small harness that
    baseline/build_ref_gpu.py compiles into the git-ignored baseline/_ref/.  Not the reference arm (that stays
    the CPU path); `unavailable` with the reason if the harness was not built or does not run."""
    exe = os.path.join(REPO, "baseline", "_ref", "ref_lutgemm_bench")
    if not os.path.exists(exe):
        return {"unavailable": "baseline/_ref/ref_lutgemm_bench not built (python baseline/build_ref_gpu.py needs the reference sources)"}
    try:
        res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    except (OSError, subprocess.TimeoutExpired) as exc:
        return {"unavailable": f"harness did not run: {type(exc).__name__}"}
    if res.returncode != 0:
        return {"unavailable": f"harness exited {res.returncode}: {res.stderr.strip()[-200:]}"}
    try:
        return json.loads(res.stdout.strip().splitlines()[-1])
    except (ValueError, IndexError):
        return {"unavailable": "harness printed no JSON line"}


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: dequantise (once, as the reference does at load) + fp32 matmul
# ------------------------------------------------------------------------------------------
def cpu_reference(workload, sample_layers=1, reps=5):
    """Times the reference's CPU path on a bounded sample: the 7 linears of `sample_layers`
    decoder blocks.  Dequantisation (lut_gemm/kernel.py:26-56 semantics, via the oracle port)
    happens once per layer, as the reference does when it loads a checkpoint
    (lut_gemm/kernel.py:101-107); the timed steady state is x.float() @ W.T in fp32 with all
    host threads."""
    from oracle import bcq_oracle as oracle
    from shiftaddllm_b200 import synth

    _, q, groups = WORKLOADS[workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    mats, nbytes, t_deq = [], 0, 0.0
    for li in range(sample_layers):
        for grp in groups:
            for _, k, n in grp:
                layer = synth.make_layer(k, n, q, G, packed_draw=True, layer_index=li)
                t0 = time.perf_counter()
                w = oracle.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
                t_deq += time.perf_counter() - t0
                mats.append((torch.from_numpy(w), layer.x.float()))
                nbytes += algorithmic_bytes(k, n, q)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        for w, x in mats:
            torch.matmul(x, w.t())
        times.append(time.perf_counter() - t0)
    t_mm = statistics.median(times)
    return {"value": round(nbytes / t_mm / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{sample_layers} decoder block(s) = {len(mats)} products, fp32 matmul median of {reps}, weights dequantised once beforehand",
            "matmul_s": round(t_mm, 5), "dequantise_s": round(t_deq, 3),
            "dequantise": "port, vectorised numpy (the reference's unpack_weight loops G x q times over the whole matrix and is far slower)",
            "value_with_dequantise": round(nbytes / (t_mm + t_deq) / 1e9, 3)}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    steps = max(args.steps, 1)
    from oracle import bcq_oracle as oracle
    from shiftaddllm_b200 import synth

    n_layers, q, groups = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    mats, nbytes = [], 0
    for grp in groups:
        for _, k, n in grp:
            layer = synth.make_layer(k, n, q, G, packed_draw=True)
            mats.append((torch.from_numpy(oracle.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())), layer.x.float()))
            nbytes += algorithmic_bytes(k, n, q)

    def step():
        for w, x in mats:
            torch.matmul(x, w.t())

    for _ in range(max(args.warmup, 3)):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = round(nbytes / dt / 1e9, 2)
    sample = ("one decoder block (7 products) per step; fp32 torch.matmul on weights dequantised once beforehand by the "
              "vectorised numpy port (reference load path)")
    return {"metric": metric_name(args.workload, q), "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(dt * 1e3, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "reference",
            "config": {"workload": f"{args.workload} decode linear set, M=1, BCQ {q}-bit g128", "sample": sample},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--legs", default=",".join(ALL_LEGS),
                    help="comma-separated sub-records to run besides the headline (default: all); 'none' for the headline alone; "
                         "'shapes' prints per-shape lines instead")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-decoder tokens/s leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: all-gather of the output slices fused into the kernel (peer stores) or a separate NCCL call")
    ap.add_argument("--workload", default="llama2-7b", choices=sorted(WORKLOADS),
                    help="linear set to run (default: the configuration the headline metric is quoted on)")
    ap.add_argument("--layers", type=int, default=None,
                    help="decoder blocks of the headline set to build (default: all of the workload); a few blocks make a small "
                         "process for profiler captures, the launches are the same")
    ap.add_argument("--shapes", default="4096x4096,4096x11008,11008x4096", help="--legs shapes: KxN list")
    ap.add_argument("--wbits", default="3", help="--legs shapes: plane counts")
    ap.add_argument("--mode", default="row", choices=["row", "block_int8"],
                    help="--legs shapes: alpha per K group and column (row), or int8 multipliers per 8 inputs x 16 outputs (block_int8)")
    ap.add_argument("--batch", default="1", help="--legs shapes: activation rows")
    args = ap.parse_args()
    args.legs = [] if args.legs == "none" else [leg for leg in args.legs.split(",") if leg]
    if args.no_decode and "decode" in args.legs:
        args.legs.remove("decode")
    if args.no_cpu_baseline and "cpu_baseline" in args.legs:
        args.legs.remove("cpu_baseline")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU: the LUT-GEMV path has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    try:
        if args.legs == ["shapes"]:
            timer = Timer(args, device, world, torch.cuda.Stream(device))
            for row in shapes_record(args, timer, device):
                print(json.dumps(row), flush=True)
        else:
            out = run_ours(args, rank, world, device)
            if out is not None:
                print(json.dumps(out), flush=True)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()

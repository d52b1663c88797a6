#!/usr/bin/env python3
"""Benchmark of the BCQ LUT-GEMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1 and N > 1 alike): the LLaMA-2-7B decode linear set at batch M = 1 —
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
inside the timed region.  `--impl reference` times the reference's CPU path (dequantise, then
fp32 matmul) on this host's cores on a bounded sample of the same workload.
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
    # the configuration the column-parallel scheme is meant for (2-bit, GQA); not the default
    "llama2-70b": (80, 2, ((("q_proj", 8192, 8192), ("k_proj", 8192, 1024), ("v_proj", 8192, 1024)),
                           (("o_proj", 8192, 8192),),
                           (("gate_proj", 8192, 28672), ("up_proj", 8192, 28672)),
                           (("down_proj", 28672, 8192),))),
}
G = 128
LAYERS, Q, GROUPS = WORKLOADS["llama2-7b"]
METRIC = "BCQ LUT-GEMV HBM GB/s, LLaMA-2-7B 3-bit g128 decode linear set, M=1"


def select_workload(name):
    global LAYERS, Q, GROUPS, METRIC
    LAYERS, Q, GROUPS = WORKLOADS[name]
    if name != "llama2-7b":
        METRIC = f"BCQ LUT-GEMV HBM GB/s, {name} {Q}-bit g128 decode linear set, M=1"


def algorithmic_bytes(k, n, q=Q, g=G, m=1):
    """Packed planes + alpha + activations (output excluded, no bias in this workload)."""
    return k * n * q // 8 + (k // g) * n * q * 2 + 2 * m * k


def step_bytes():
    return LAYERS * sum(algorithmic_bytes(k, n) for grp in GROUPS for _, k, n in grp)


def measured_peak():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.proc.wait()

    def summary(self):
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].startswith("Active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def build_model(device, rank, world, seed=0):
    """Weights of all 32 blocks (column shard of `rank`), drawn on the device from a seeded
    generator: packed words uniform in int32 (every bit i.i.d. +-1), alpha = 2**-k, k in 2..8."""
    gen = torch.Generator(device=device).manual_seed(1000003 * seed + 17)
    blocks = []
    for _ in range(LAYERS):
        groups = []
        for grp in GROUPS:
            probs = []
            for _, k, n in grp:
                n_loc = n // world
                bw = torch.randint(-2 ** 31, 2 ** 31, (k // 32, Q, n_loc), dtype=torch.int32, device=device, generator=gen)
                alpha = torch.exp2(-torch.randint(2, 9, (k // G, Q, n_loc), device=device, generator=gen).float()).half()
                probs.append({"K": k, "N": n, "N_loc": n_loc, "bw": bw, "alpha": alpha})
            groups.append(probs)
        blocks.append(groups)
    return blocks


def run_ours(args, rank, world, device):
    import torch.distributed as dist

    from shiftaddllm_b200 import _lib, lutgemm

    lib = _lib.load()
    _lib.check(lib.sal_device_ok(), "sal_device_ok")
    blocks = build_model(device, rank, world)
    gen = torch.Generator(device=device).manual_seed(4242)
    # per product: device input, device output slice, (gathered output when world > 1)
    n_in = sum(k for grp in GROUPS for _, k, _ in grp) * LAYERS
    n_out = sum(n for grp in GROUPS for _, _, n in grp) * LAYERS
    x_all = torch.randn(n_in, device=device, generator=gen).half()
    y_all = torch.zeros(n_out // world, dtype=torch.float16, device=device)
    fused = world > 1 and args.exchange == "fused"
    peer = None
    if fused:
        from shiftaddllm_b200.exchange import PeerExchange

        try:
            peer = PeerExchange.symmetric(n_out, nslots=4)
            ok = torch.ones(1, device=device)
        except Exception as exc:  # noqa: BLE001 - no peer-mappable memory on this box: use NCCL on every rank
            print(f"[bench] symmetric memory unavailable ({type(exc).__name__}: {exc}); using the NCCL exchange", file=sys.stderr)
            ok = torch.zeros(1, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)   # all ranks take the same path
        fused = bool(ok.item())
    if fused:
        y_full = peer.buffer
    else:
        y_full = torch.zeros(n_out, dtype=torch.float16, device=device) if world > 1 else None
    def make_launches(per_block_groups):
        """per_block_groups: lists of product indices (0..6 within a block) sharing one launch."""
        launches = []
        xi = yi = yfi = 0
        for groups in blocks:
            flat = [p for probs in groups for p in probs]
            views = []
            for p in flat:
                views.append((x_all[xi:xi + p["K"]].view(1, -1), y_all[yi:yi + p["N_loc"]].view(1, -1), yi))
                xi += p["K"]
                yi += p["N_loc"]
            for idxs in per_block_groups:
                plist = []
                for i in idxs:
                    p, (x, y, _) = flat[i], views[i]
                    plist.append(dict(output=y, bWeight=p["bw"], alpha=p["alpha"], bias=None, d_input=x,
                                      mSize=p["N_loc"], kSize=p["K"], nb=Q, num_groups=p["K"] // G))
                gathered = None
                if world > 1:   # the launch's output slices are contiguous in y_all: one exchange per launch
                    lo = views[idxs[0]][2]
                    hi = views[idxs[-1]][2] + flat[idxs[-1]]["N_loc"]
                    if fused:   # every product owns a [world][N_loc] block of the gather buffer
                        offs = []
                        for i in idxs:
                            offs.append(yfi)
                            yfi += flat[i]["N"]
                        gathered = offs
                    else:
                        gathered = (y_full[yfi:yfi + (hi - lo) * world], y_all[lo:hi])
                        yfi += (hi - lo) * world
                launches.append((plist, gathered))
        return launches

    def make_step(launches):
        # argument blocks are validated and marshalled once; a step then only enqueues
        prepared = None if fused else [lutgemm.prepare_grouped(plist, pdl=True) for plist, _ in launches]

        def one_step():
            for li, (plist, gathered) in enumerate(launches):
                if fused:
                    writers = peer.launch(plist, gathered, li % 4, pdl=True)
                    peer.wait(li % 4, writers)
                else:
                    prepared[li]()
                    if gathered is not None:
                        dist.all_gather_into_tensor(gathered[0], gathered[1])
        return one_step

    stream = torch.cuda.Stream(device)

    def capture(one_step):
        with torch.cuda.stream(stream):
            one_step()                       # also sizes the workspace and runs the one-off probes
            torch.cuda.synchronize(device)
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    one_step()
                return g.replay, True
            except Exception as exc:  # noqa: BLE001 - a failed capture (e.g. of a collective) falls back to eager launches
                print(f"[bench] graph capture failed ({type(exc).__name__}); timing eager launches", file=sys.stderr)
                torch.cuda.synchronize(device)
                return one_step, False

    launches = make_launches([[0, 1, 2, 3, 4, 5, 6]])
    one_step = make_step(launches)
    replay, graphed = capture(one_step)
    dep_launches = make_launches([[0, 1, 2], [3], [4, 5], [6]])
    dep_replay, _ = capture(make_step(dep_launches))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, steps, sample_clocks=False):
        with torch.cuda.stream(stream):
            for _ in range(max(args.warmup, 3)):
                fn()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(device.index) as clk:
                e0.record(stream)
                for _ in range(steps):
                    fn()
                e1.record(stream)
                barrier()
            ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps, clk

    ms_per_step, clk = timed(replay, args.steps)
    dep_ms_per_step, _ = timed(dep_replay, max(3, args.steps // 4))

    # ---- end to end: host activations in, host results out, through the public Python API
    x_host = x_all.cpu().pin_memory()
    y_src = y_full if world > 1 else y_all
    y_host = torch.empty(y_src.shape, dtype=torch.float16).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))
    with torch.cuda.stream(stream):
        def e2e_step():
            x_all.copy_(x_host, non_blocking=True)
            one_step()
            y_host.copy_(y_src, non_blocking=True)
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_s], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    with torch.cuda.stream(stream):   # the workspace is cached per (device, stream)
        ws = lutgemm.workspace_for(device, 1, 8)
    status = lib.sal_workspace_status(ws.data_ptr(), stream.cuda_stream)

    if rank != 0:
        return None
    total = step_bytes()
    peak, which = measured_peak()
    n_launch = len(launches)
    per_launch_us = ms_per_step * 1e3 / n_launch
    achieved = total / world / (ms_per_step * 1e-3) / 1e9   # per GPU: this rank's bytes over the step time
    out = {
        "metric": METRIC, "value": round(total / (ms_per_step * 1e-3) / 1e9, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16 in, fp32 accumulate",
        "data": "synthetic", "impl": "ours",
        "config": {"workload": f"{args.workload} decode linear set ({LAYERS} blocks x 7 linears), M=1, BCQ {Q}-bit g128",
                   "launches_per_step": n_launch,
                   "launch_structure": ("one grouped launch per decoder block (7 independent products); PDL chained; "
                                        + ("CUDA graph" if graphed else "eager")),
                   "l2": f"inputs larger than L2 ({total / 1e9:.1f} GB of weights per step), no flush",
                   "parallelism": (f"column-parallel x{world}, all-gather "
                                   + ("fused into the kernel (peer-to-peer stores + counters)" if fused else "by NCCL"))
                   if world > 1 else "single GPU"},
        "tokens_per_s_linears_only": round(1e3 / ms_per_step, 1),
        "gemv_per_s": round(LAYERS * 7 * 1e3 / ms_per_step, 1),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "peak_source": f"{which} copy bandwidth (MEASURED_PEAKS.json)" if which == "measured" else "fallback 6650",
                     "kernel": f"lutgemv_tiled_kernel<{Q},8>", "avg_launch_us": round(per_launch_us, 3),
                     "algorithmic_bytes_per_launch": total // world // n_launch,
                     "traffic": read_traffic() if (args.workload == "llama2-7b" and world == 1) else None},
        "e2e": {"value": round(total / e2e_s / 1e9, 1), "unit": "GB/s", "ms_per_step": round(e2e_s * 1e3, 3),
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                "api": ("shiftaddllm_b200.lutgemm.prepare_grouped launches called eagerly from Python (no graph), "
                        "pinned host buffers, activations copied in and results copied out every step")},
        "dependency_ordered": {"launches_per_step": len(dep_launches), "ms_per_step": round(dep_ms_per_step, 4),
                               "value": round(total / (dep_ms_per_step * 1e-3) / 1e9, 1), "unit": "GB/s",
                               "structure": "per block: grouped{q,k,v}, o, grouped{gate,up}, down; PDL chained"},
        "gpu_launches": n_launch * args.steps,
        "device_status": status,
        "clocks": clk.summary(),
    }
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_reference(sample_layers=1, reps=5)
    if world == 1 and not args.no_decode:
        del launches, dep_launches, blocks
        torch.cuda.empty_cache()
        out["decode"] = decode_tokens_per_s(args.workload, device)
    return out


def decode_tokens_per_s(workload, device):
    """The other half of the metric: greedy batch-1 decode of a whole decoder of the workload's
    architecture (random init, every linear a synthetic BCQ layer): 128 new tokens after a
    512-token prompt (1024 for the 70B shape), the step replayed as one CUDA graph.  Reported for
    fixed-order fp16 GEMV outputs and for the opt-in fp32 atomic accumulation; for the 7B shape also 16
    sequences decoded in lock step (64 new tokens each) on the small-batch kernel."""
    from shiftaddllm_b200 import decoder

    prompt = 512 if workload == "llama2-7b" else 1024
    with torch.cuda.device(device):
        model = decoder.BcqLlamaDecoder(decoder.SHAPES[workload], Q, G, max_len=prompt + 2 * 128 + 16, device=device)
        res = {}
        for name, atomic in (("fp16_outputs", False), ("f32_atomic_outputs", True)):
            model.set_atomic(atomic)
            r = decoder.benchmark(model, prompt, 128)
            res[name] = {"tokens_per_s": round(r["tokens_per_s"], 1), "ms_per_token": round(r["ms_per_token"], 4),
                         "median_ms_per_token_synced": round(r["median_ms_per_token_synced"], 4)}
        if workload == "llama2-7b":
            # 16 sequences in lock step: the linears run the small-batch (M = 16) LUT kernel
            batch = decoder.BcqLlamaBatchDecoder(decoder.SHAPES[workload], Q, G, max_len=prompt + 64 + 16, batch=16, device=device,
                                                 like=model)
            r = decoder.benchmark_batch(batch, prompt, 64)
            res["batch16_fp16_outputs"] = {"tokens_per_s": round(r["tokens_per_s"], 1), "ms_per_step": round(r["ms_per_step"], 3),
                                           "new_tokens_per_sequence": 64}
    res["workload"] = (f"{workload}-shaped decoder, BCQ {Q}-bit g128 linears, fp16 lm_head, batch 1, {prompt}-token prompt of "
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


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: dequantise (once, as the reference does at load) + fp32 matmul
# ------------------------------------------------------------------------------------------
def cpu_reference(sample_layers=1, reps=5):
    """Times the reference's CPU path on a bounded sample: the 7 linears of `sample_layers`
    decoder blocks.  Dequantisation (lut_gemm/kernel.py:26-56 semantics, via the oracle port)
    happens once per layer, as the reference does when it loads a checkpoint
    (lut_gemm/kernel.py:101-107); the timed steady state is x.float() @ W.T in fp32 with all
    host threads."""
    from oracle import bcq_oracle as oracle
    from shiftaddllm_b200 import synth

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    mats, nbytes, t_deq = [], 0, 0.0
    for li in range(sample_layers):
        for grp in GROUPS:
            for _, k, n in grp:
                layer = synth.make_layer(k, n, Q, G, packed_draw=True, layer_index=li)
                t0 = time.perf_counter()
                w = oracle.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())
                t_deq += time.perf_counter() - t0
                mats.append((torch.from_numpy(w), layer.x.float()))
                nbytes += algorithmic_bytes(k, n)
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
            "value_with_dequantise": round(nbytes / (t_mm + t_deq) / 1e9, 3)}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    steps = max(args.steps, 1)
    from oracle import bcq_oracle as oracle
    from shiftaddllm_b200 import synth

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    mats, nbytes = [], 0
    for grp in GROUPS:
        for _, k, n in grp:
            layer = synth.make_layer(k, n, Q, G, packed_draw=True)
            mats.append((torch.from_numpy(oracle.dequant_mode_a(layer.bWeight.numpy(), layer.alpha.numpy())), layer.x.float()))
            nbytes += algorithmic_bytes(k, n)

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
    sample = "one decoder block (7 products) per step; fp32 torch.matmul on weights dequantised once beforehand (reference load path)"
    return {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(dt * 1e3, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32", "data": "synthetic", "impl": "reference",
            "config": {"workload": f"{args.workload} decode linear set, M=1, BCQ {Q}-bit g128", "sample": sample},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-decoder tokens/s leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: all-gather of the output slices fused into the kernel (peer stores) or a separate NCCL call")
    ap.add_argument("--workload", default="llama2-7b", choices=sorted(WORKLOADS),
                    help="linear set to run (default: the configuration the headline metric is quoted on)")
    args = ap.parse_args()
    select_workload(args.workload)

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
        out = run_ours(args, rank, world, device)
        if out is not None:
            print(json.dumps(out), flush=True)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Per-shape timing of the mode-A LUT-GEMV / small-batch product.

    python -m shiftaddllm_b200.microbench --shapes 4096x4096,4096x11008 --wbits 2,3,4 --batch 1,4,8,16,64

Each (shape, wbits, M) is timed over a rotation of distinct weight tensors whose total size
exceeds the L2 cache (so every call streams its weights from HBM), as one CUDA graph of
back-to-back launches chained with programmatic dependent launch, with CUDA events.
Prints one JSON line per case: microseconds per call, algorithmic GB/s
(planes + alpha + activations; output excluded) and the fraction of `--peak` GB/s.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import lutgemm


def algorithmic_bytes(k, n, q, g, m):
    return k * n * q // 8 + (k // g) * n * q * 2 + 2 * m * k


def time_case(k, n, q, g, m, peak, min_total_bytes=256 << 20, reps=5, device="cuda"):
    per = k * n * q // 8
    copies = max(4, min(64, -(-min_total_bytes // per)))
    gen = torch.Generator(device=device).manual_seed(k * 31 + n * 7 + q)
    bws = [torch.randint(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=torch.int32, device=device, generator=gen)
           for _ in range(copies)]
    alpha = torch.exp2(-torch.randint(2, 9, (k // g, q, n), device=device, generator=gen).float()).half()
    x = torch.randn(m, k, device=device, generator=gen).half()
    y = torch.empty(m, n, dtype=torch.float16, device=device)

    def run():
        for bw in bws:
            lutgemm.lutgemv_fused(y, bw, alpha, None, x, n, k, q, k // g, pdl=True)

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
    nbytes = algorithmic_bytes(k, n, q, g, m)
    gbs = nbytes / us / 1e3
    return {"K": k, "N": n, "wbits": q, "group": g, "M": m, "us_per_call": round(us, 3), "algorithmic_bytes": nbytes,
            "GBps": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4), "weights_rotated": copies}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="768x768,4096x4096,4096x11008,11008x4096", help="KxN list")
    ap.add_argument("--wbits", default="3")
    ap.add_argument("--batch", default="1")
    ap.add_argument("--groupsize", type=int, default=128)
    ap.add_argument("--peak", type=float, default=6547.2, help="GB/s the fraction is taken of")
    args = ap.parse_args()
    for shape in args.shapes.split(","):
        k, n = (int(v) for v in shape.lower().split("x"))
        for q in (int(v) for v in args.wbits.split(",")):
            for m in (int(v) for v in args.batch.split(",")):
                print(json.dumps(time_case(k, n, q, args.groupsize, m, args.peak)), flush=True)


if __name__ == "__main__":
    main()

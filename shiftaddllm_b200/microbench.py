"""Per-shape timing of the LUT-GEMV / small-batch product.

    python -m shiftaddllm_b200.microbench --shapes 4096x4096,4096x11008 --wbits 2,3,4 --batch 1,4,8,16,64
    python -m shiftaddllm_b200.microbench --mode block_int8 --shapes 4096x4096     # block layouts (alpha [K/8][q][N/16])

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


ALPHA_BYTES = {"row": 2, "block": 2, "block_shift": 2, "block_int8": 3}


def algorithmic_bytes(k, n, q, g, m, mode="row"):
    # alpha: one value per (g inputs, plane, column) in row mode, per (8 inputs, plane, g/8 columns) in the block modes:
    # the same count of values either way
    return k * n * q // 8 + (k // g) * n * q * ALPHA_BYTES[mode] + 2 * m * k


def time_case(k, n, q, g, m, peak, min_total_bytes=256 << 20, reps=5, device="cuda", mode="row"):
    per = k * n * q // 8
    copies = max(4, min(64, -(-min_total_bytes // per)))
    gen = torch.Generator(device=device).manual_seed(k * 31 + n * 7 + q)
    bws = [torch.randint(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=torch.int32, device=device, generator=gen)
           for _ in range(copies)]
    x = torch.randn(m, k, device=device, generator=gen).half()
    y = torch.empty(m, n, dtype=torch.float16, device=device)
    if mode == "row":
        alpha = torch.exp2(-torch.randint(2, 9, (k // g, q, n), device=device, generator=gen).float()).half()

        def run():
            for bw in bws:
                lutgemm.lutgemv_fused(y, bw, alpha, None, x, n, k, q, k // g, pdl=True)
    else:
        ng = n // (g // 8)          # columns per multiplier = groupsize / 8 (16 at g128)
        if mode == "block":
            alpha = torch.exp2(-torch.randint(2, 9, (k // 8, q, ng), device=device, generator=gen).float()).half()
        elif mode == "block_shift":
            alpha = torch.randint(0, 512, (k // 8, q, ng), device=device, generator=gen).to(torch.int16)
            x = x * 0.01            # multipliers reach 384
        else:
            alpha = torch.randint(-9, -1, (k // 8, q, ng, 3), device=device, generator=gen).to(torch.int8)

        def run():
            for bw in bws:
                lutgemm.lutgemm_block_fused(y, bw, alpha, None, x, n, k, q, ng, pdl=True)

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
    nbytes = algorithmic_bytes(k, n, q, g, m, mode)
    gbs = nbytes / us / 1e3
    return {"mode": mode, "K": k, "N": n, "wbits": q, "group": g, "M": m, "us_per_call": round(us, 3), "algorithmic_bytes": nbytes,
            "GBps": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4), "weights_rotated": copies}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="768x768,4096x4096,4096x11008,11008x4096", help="KxN list")
    ap.add_argument("--wbits", default="3")
    ap.add_argument("--batch", default="1")
    ap.add_argument("--groupsize", type=int, default=128)
    ap.add_argument("--mode", default="row", choices=sorted(ALPHA_BYTES), help="alpha layout / multiplier encoding")
    ap.add_argument("--peak", type=float, default=6547.2, help="GB/s the fraction is taken of")
    args = ap.parse_args()
    for shape in args.shapes.split(","):
        k, n = (int(v) for v in shape.lower().split("x"))
        for q in (int(v) for v in args.wbits.split(",")):
            for m in (int(v) for v in args.batch.split(",")):
                print(json.dumps(time_case(k, n, q, args.groupsize, m, args.peak, mode=args.mode)), flush=True)


if __name__ == "__main__":
    main()

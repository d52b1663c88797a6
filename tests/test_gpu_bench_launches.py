"""The launches `bench.py` times, checked against the oracle.

The work split of a grouped launch depends on the whole shape set of the launch (a CTA may start and
end in the middle of a K block, ranges of one problem may have different numbers of K splits), so the
7-product decoder-block launch and the four dependency-ordered groups are different plans from any
single-product call.  These tests build exactly those launches through the benchmark's own builder
(two decoder blocks are enough: the plan of a launch depends only on its own shapes) and compare EVERY
product's output with the dequantise oracle on a sample of output columns: both sides of every
256-column tile boundary (column ranges are whole tiles), the first and last columns — the 11008 and
28672 tails included — and seeded random columns.  The oracle is exact on the columns it is given.

Tolerance: max|y - ref| / max|ref| <= 1e-2 (the bar stated for fp16 accumulation; measured ~5e-4).
"""
import ctypes

import numpy as np
import pytest
import torch

import bench
from oracle import bcq_oracle as o
from shiftaddllm_b200 import _lib, lutgemm

pytestmark = pytest.mark.gpu
TOL = 1e-2


def oracle_columns(p, cols):
    """Oracle output of product `p` (a bench.LinearSet entry) on the columns `cols`."""
    idx = torch.tensor(cols, device=p["bw"].device)
    bw = p["bw"][:, :, idx].cpu().numpy()
    x = p["x"].cpu().numpy()
    if p["alpha"].dtype == torch.float16:
        w = o.dequant_mode_a(bw, p["alpha"][:, :, idx].cpu().numpy())
    else:   # block layout: one int8 exponent triple per 8 inputs x 16 outputs; expand the multipliers per column
        mult = o.apot_i8_multiplier(p["alpha"].cpu().numpy())                        # [K/8, q, N/16]
        per_col = mult[:, :, np.asarray(cols) // bench.BLOCK_GS]                      # [K/8, q, C]
        w = o.dequant_mode_b(bw, per_col)                                            # groups of one column
    return o.linear_fp32(x, w)


def check_products(products):
    worst = 0.0
    for p in products:
        cols = bench.sample_columns(p["N_loc"], count=256)
        got = p["y"][:, torch.tensor(cols, device=p["y"].device)].float().cpu().numpy()
        err = o.max_rel_err(got, oracle_columns(p, cols))
        assert err <= TOL, f"{p['K']}x{p['N']} q{p['q']}: max relative error {err}"
        worst = max(worst, err)
    return worst


def status_clean():
    lib = _lib.load()
    ws = lutgemm.workspace_for(torch.device("cuda", torch.cuda.current_device()), 1, 8)
    return lib.sal_workspace_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0


@pytest.mark.parametrize("workload", ["llama2-7b", "llama2-70b"])
@pytest.mark.parametrize("groups", [bench.HEADLINE_GROUPS, bench.DEPENDENCY_GROUPS], ids=["block_launch", "dependency_ordered"])
def test_timed_launches_match_the_oracle(workload, groups):
    dev = torch.device("cuda", 0)
    lset = bench.LinearSet(workload, dev, layers=2)
    run = bench.SetRunner(lset, groups)
    run.step()
    torch.cuda.synchronize()
    check_products([p for prods in run.products for p in prods])
    assert status_clean()
    # the benchmark replays the step as a CUDA graph: same launches, bit-identical results
    eager = lset.y_all.clone()
    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        run.step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run.step()
    lset.y_all.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(lset.y_all, eager)
    assert bench.verify_products(run.products[0], dev) <= TOL      # the benchmark's own checker agrees with the oracle


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 11008), (11008, 4096)])
@pytest.mark.parametrize("q", [2, 3, 4])
def test_small_batch_on_the_7b_shapes(k, n, q):
    """The mixed-precision small-batch configuration on its own shapes: M in {4, 8, 16, 64} (and an odd
    M), every width the configuration draws from, incl. the 11008 column tail (43 tiles)."""
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(k + 3 * n + q)
    bw = torch.randint(-2 ** 31, 2 ** 31, (k // 32, q, n), dtype=torch.int32, device=dev, generator=gen)
    alpha = torch.exp2(-torch.randint(2, 9, (k // 128, q, n), device=dev, generator=gen).float()).half()
    for m in (4, 7, 8, 16, 64):
        x = torch.randn(m, k, device=dev, generator=gen).half()
        y = torch.empty(m, n, dtype=torch.float16, device=dev)
        lutgemm.lutgemv_fused(y, bw, alpha, None, x, n, k, q, k // 128, pdl=True)
        torch.cuda.synchronize()
        check_products([{"K": k, "N": n, "N_loc": n, "q": q, "bw": bw, "alpha": alpha, "x": x, "y": y}])
    assert status_clean()


@pytest.mark.parametrize("m", [1, 4, 16])
def test_mixed_bit_widths_in_one_grouped_launch(m):
    """Per-layer widths drawn from {2,3,4}: the products of one decoder block in ONE grouped call
    (issued as one kernel per distinct width)."""
    dev = torch.device("cuda", 0)
    bits = bench.mixed_bits(14, seed=1)
    assert len(set(bits[:7])) > 1
    lset = bench.LinearSet("llama2-7b", dev, layers=2, bits=bits, m=m, seed=2)
    run = bench.SetRunner(lset, bench.HEADLINE_GROUPS)
    run.step()
    torch.cuda.synchronize()
    check_products([p for prods in run.products for p in prods])
    # the one-off form of the same call
    for flat in lset.blocks:
        lset.y_all.zero_()
        lutgemm.lutgemv_grouped([lset.problem(p) for p in flat], pdl=True)
        torch.cuda.synchronize()
        check_products(flat)
    assert status_clean()


def test_block_layout_launches_of_the_benchmark():
    dev = torch.device("cuda", 0)
    lset = bench.LinearSet("llama2-7b", dev, layers=1, layout="block_int8", seed=7)
    for p in lset.blocks[0]:
        lutgemm.lutgemm_block_fused(p["y"], p["bw"], p["alpha"], None, p["x"], p["N"], p["K"], p["q"], p["N"] // bench.BLOCK_GS, pdl=True)
    torch.cuda.synchronize()
    check_products(lset.blocks[0])
    assert bench.verify_products(lset.blocks[0], dev) <= TOL
    assert status_clean()


@pytest.mark.parametrize("k,n", [(8192, 8192), (8192, 28672), (28672, 8192), (8192, 1024)])
def test_config5_shapes_single_products(k, n):
    """The 70B shapes (2 bit) one product per launch, as a column-parallel rank at 1 GPU issues them."""
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(k + n)
    bw = torch.randint(-2 ** 31, 2 ** 31, (k // 32, 2, n), dtype=torch.int32, device=dev, generator=gen)
    alpha = torch.exp2(-torch.randint(2, 9, (k // 128, 2, n), device=dev, generator=gen).float()).half()
    for m in (1, 16):
        x = torch.randn(m, k, device=dev, generator=gen).half()
        y = torch.empty(m, n, dtype=torch.float16, device=dev)
        lutgemm.lutgemv_fused(y, bw, alpha, None, x, n, k, 2, k // 128, pdl=True)
        torch.cuda.synchronize()
        check_products([{"K": k, "N": n, "N_loc": n, "q": 2, "bw": bw, "alpha": alpha, "x": x, "y": y}])
    assert status_clean()


def test_prepared_launch_through_the_c_abi():
    """sal_prepare_grouped + sal_launch_prepared give bit-identical results to sal_lutgemv_grouped, launch
    after launch, and refuse a scratch buffer that is too small."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    lset = bench.LinearSet("llama2-7b", dev, layers=1, seed=4)
    flat = lset.blocks[0]
    arr, keep = lutgemm.marshal_problems([lset.problem(p) for p in flat])
    stream = torch.cuda.current_stream().cuda_stream
    ws = lutgemm.workspace_for(dev, 1, sum(p["N"] for p in flat))
    assert lib.sal_lutgemv_grouped(arr, len(flat), 0, ws.data_ptr(), ws.numel(), stream) == 0
    torch.cuda.synchronize()
    want = lset.y_all.clone()
    handle = ctypes.c_void_p()
    assert lib.sal_prepare_grouped(arr, len(flat), 0, None, ctypes.byref(handle)) == 0
    need = lib.sal_prepared_workspace_bytes(handle)
    assert 16384 <= need <= ws.numel()
    for _ in range(2):
        lset.y_all.zero_()
        assert lib.sal_launch_prepared(handle, ws.data_ptr(), ws.numel(), -1, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(lset.y_all, want)
    assert lib.sal_launch_prepared(handle, ws.data_ptr(), 1024, -1, stream) == _lib.SAL_E_WORKSPACE
    # several prepared launches enqueued by one call
    second = ctypes.c_void_p()
    assert lib.sal_prepare_grouped(arr, len(flat), _lib.SAL_PDL, None, ctypes.byref(second)) == 0      # same problems: same plan
    handles = (ctypes.c_void_p * 2)(handle, second)
    lset.y_all.zero_()
    assert lib.sal_launch_prepared_sequence(handles, 2, None, ws.data_ptr(), ws.numel(), stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(lset.y_all, want)
    lib.sal_destroy_prepared(handle)
    lib.sal_destroy_prepared(second)
    check_products(flat)


def test_two_stream_issue_gives_the_same_results():
    """The benchmark's `overlapped_launches` arm (even launches on one stream, odd ones on a second, each with its own
    scratch buffer) computes what the single-stream step computes, bit for bit, eagerly and from a captured graph."""
    dev = torch.device("cuda", 0)
    lset = bench.LinearSet("llama2-7b", dev, layers=4, seed=3)
    run = bench.SetRunner(lset, bench.HEADLINE_GROUPS)
    main, side = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    with torch.cuda.stream(main):
        run.step()
        torch.cuda.synchronize()
        want = lset.y_all.clone()
        lset.y_all.zero_()
        run.step_two_streams(side)
        torch.cuda.synchronize()
        assert torch.equal(lset.y_all, want)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=main):
            run.step_two_streams(side)
        lset.y_all.zero_()
        graph.replay()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(lset.y_all, want)
    check_products([p for prods in run.products for p in prods])
    assert status_clean()

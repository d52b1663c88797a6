"""B200-native BCQ LUT-GEMV: a drop-in for ShiftAddLLM's ``lut_gemm`` path.

* :mod:`shiftaddllm_b200.lutgemm`  — the compiled extension's API (five entry points)
* :mod:`shiftaddllm_b200.quant`    — ``LutLinear``, ``make_lut``, ``load_lut``
* :mod:`shiftaddllm_b200.kernel`   — pack / unpack / convert / checkpoint loaders
* :mod:`shiftaddllm_b200.shard`    — column-parallel partition + all-gather
* :mod:`shiftaddllm_b200.synth`    — seeded synthetic layers of the benchmark shapes
"""
__version__ = "0.1.0"

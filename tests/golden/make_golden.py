"""Generate ``tests/golden/reference_vectors.npz`` from the UNMODIFIED reference.

Run where a checkout of GATECH-EIC/ShiftAddLLM is available:

    python tests/golden/make_golden.py --reference <path-to-ShiftAddLLM>

The reference's ``lut_gemm/quant.py`` imports its compiled ``lutgemm`` extension
at module import; an empty stand-in module is registered first, nothing from it
is called.  All inputs are drawn from seeded CPU generators, all outputs are
what the reference's own functions return on CPU:

* ``pack_binaryWeight``            (lut_gemm/kernel.py:9-23)
* ``unpack_weight``                (lut_gemm/kernel.py:26-56)
* ``unpack_to_fake_binaryWeight``  (lut_gemm/kernel.py:58-75)
* ``convert_weight`` (square case) (lut_gemm/kernel.py:112-133)
* ``LutLinear.quantize_to_apot``   (lut_gemm/quant.py:30-39)
* the dequantise-then-matmul layer output, fp32 (lut_gemm/kernel.py:101-107)
"""
import argparse
import os
import sys
import types

import numpy as np
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of an unmodified checkout of GATECH-EIC/ShiftAddLLM")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz"))
    args = ap.parse_args()

    sys.path.insert(0, args.reference)
    sys.modules.setdefault("lutgemm", types.ModuleType("lutgemm"))
    from lut_gemm.kernel import (convert_weight, pack_binaryWeight, unpack_to_fake_binaryWeight, unpack_weight)
    from lut_gemm.quant import LutLinear

    out = {}
    gen = torch.Generator().manual_seed(20240611)

    def planes(*shape):
        return torch.randint(0, 2, shape, generator=gen, dtype=torch.int64) * 2 - 1

    # --- pack / unpack, three shapes (last one has bit 31 set everywhere in plane 0)
    for tag, shape in (("p0", (8, 2, 64, 3)), ("p1", (5, 1, 32, 1)), ("p2", (12, 3, 128, 4))):
        b = planes(*shape)
        if tag == "p1":
            b[:, :, 31, 0] = 1
        packed = pack_binaryWeight(b.float())
        alpha = torch.rand(shape[0], shape[1], shape[3], generator=gen) + 0.05
        w = unpack_weight(packed, alpha)
        fake = unpack_to_fake_binaryWeight(packed, n_groups=shape[1])
        out[f"{tag}_planes"] = b.to(torch.int8).numpy()
        out[f"{tag}_packed"] = packed.numpy()
        out[f"{tag}_alpha"] = alpha.numpy()
        out[f"{tag}_weight"] = w.numpy()
        out[f"{tag}_fake_u8"] = fake.numpy()
        # the reference's own self-check: pack -> unpack equals einsum(B, alpha)
        q = torch.einsum("nijl,nil->nij", b.float(), alpha).flatten(1)
        out[f"{tag}_einsum"] = q.numpy()

    # --- convert_weight on a square Lat.-style layer (K_in = N_out = 64)
    k_in = n_out = 64
    q = 3
    gs = 16
    b_lat = planes(k_in, n_out // gs, gs, q)  # [K_in, N/gs, gs, q], packed along N
    packed_lat = pack_binaryWeight(b_lat.float())  # [K_in, N/32, q]
    alpha_blk = torch.rand(k_in // 8, n_out // gs, q, generator=gen) + 0.05
    alpha_rep = alpha_blk.repeat_interleave(8, dim=0)
    conv_bw, conv_alpha = convert_weight(packed_lat, alpha_rep)
    w_t = unpack_weight(packed_lat, alpha_rep)  # [K_in, N_out] = W^T
    out["cv_planes"] = b_lat.to(torch.int8).numpy()
    out["cv_packed_lat"] = packed_lat.numpy()
    out["cv_alpha_blk"] = alpha_blk.numpy()
    out["cv_kernel_bw"] = conv_bw.numpy()
    out["cv_kernel_alpha"] = conv_alpha.numpy()
    out["cv_weight_t"] = w_t.numpy()

    # --- APoT exponents
    lin = LutLinear(32, 32, 32, 3, None)
    vals = torch.tensor([0.25, 2.0 ** -7, 0.3, 0.011, 1.7, -0.3, 0.0625, 0.7071, 3.3, 0.0009765625, 0.19, 5e-3],
                        dtype=torch.float32)
    rnd = torch.rand(64, generator=gen) * 0.5 + 1e-3
    apot_in = torch.cat([vals, rnd])
    out["apot_in"] = apot_in.numpy()
    out["apot_out"] = lin.quantize_to_apot(apot_in.clone()).numpy()

    # --- mode A layer: planes [N, K/g, g, q] -> packed [N, K/32, q]; alpha = 2^-k
    n, k, g, q = 64, 256, 128, 3
    b = planes(n, k // g, g, q)
    packed = pack_binaryWeight(b.float())
    kexp = torch.randint(2, 9, (n, k // g, q), generator=gen)
    alpha = (2.0 ** (-kexp.float())).half()
    x = torch.randn(1, k, generator=gen).half()
    bias = (0.02 * torch.randn(n, generator=gen)).half()
    w = unpack_weight(packed, alpha.float())
    y = x.float() @ w.t() + bias.float()
    out["la_packed"] = packed.numpy()
    out["la_alpha_f16"] = alpha.numpy()
    out["la_x_f16"] = x.numpy()
    out["la_bias_f16"] = bias.numpy()
    out["la_weight"] = w.numpy()
    out["la_y"] = y.numpy()

    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()

"""The per-layer "Lat." checkpoint format of the reference
(`{dir}/{model}_{i}.{name}_{wbits}bit.pt` holding `bWeight [K_in, N_out/32, wbits]` packed along
out_features and `alpha [K_in/8, N_out/gs, wbits]`; quant_methods/shiftaddllm.py:191-211) read
into a tiny randomly initialised HF OPT, both ways the reference offers: dense "simulation"
weights (lut_gemm/kernel.py:87-109) and LutLinear modules (lut_gemm/kernel.py:135-179)."""
import numpy as np
import pytest
import torch

from oracle import bcq_oracle as o
from shiftaddllm_b200 import kernel as K
from shiftaddllm_b200.quant import LutLinear

transformers = pytest.importorskip("transformers")
WBITS, GS = 3, 16   # gs = groupsize / 8 = 16 columns per alpha block (groupsize 128)


def tiny_opt():
    cfg = transformers.OPTConfig(hidden_size=128, ffn_dim=256, num_hidden_layers=2, num_attention_heads=4, vocab_size=512,
                                 max_position_embeddings=64, word_embed_proj_dim=128, dropout=0.0)
    torch.manual_seed(0)
    return transformers.OPTForCausalLM(cfg).half().eval()


def write_checkpoints(model, directory, name="opt-tiny"):
    gen = torch.Generator().manual_seed(7)
    dense = {}
    for i, layer in enumerate(model.model.decoder.layers):
        for lname, lin in K.find_layers(layer).items():
            k_in, n_out = lin.in_features, lin.out_features
            planes = torch.randint(0, 2, (k_in, n_out // GS, GS, WBITS), generator=gen, dtype=torch.int8) * 2 - 1
            alpha = torch.exp2(-torch.randint(3, 8, (k_in // 8, n_out // GS, WBITS), generator=gen).float())
            # the product-side writer (quant_methods/shiftaddllm.py:191-211): packs along out_features, saves
            path = K.save_lat_checkpoint(planes, alpha, str(directory), name, f"{i}.{lname}", WBITS)
            assert path == f"{directory}/{name}_{i}.{lname}_{WBITS}bit.pt"
            packed = torch.load(path)["bWeight"]                                 # [K_in, N_out/32, q]
            assert packed.dtype == torch.int32 and tuple(packed.shape) == (k_in, n_out // 32, WBITS)
            w_t = o.unpack_weight(packed.numpy(), np.repeat(alpha.numpy(), 8, axis=0))   # [K_in, N_out] via the oracle
            dense[(i, lname)] = torch.from_numpy(np.ascontiguousarray(w_t.T))
    return dense


def test_dense_simulation_load(tmp_path):
    model = tiny_opt()
    dense = write_checkpoints(model, tmp_path)
    K.load_shiftaddllm_weight(model, str(tmp_path), "opt-tiny", WBITS, is_lat=True)
    for i, layer in enumerate(model.model.decoder.layers):
        for lname, lin in K.find_layers(layer).items():
            assert torch.equal(lin.weight.data.float(), dense[(i, lname)].half().float())
    with pytest.raises(ValueError):
        K.load_shiftaddllm_weight(model, str(tmp_path), "opt-tiny", WBITS, is_lat=False)


def test_kernel_load_builds_lutlinear_with_converted_layout(tmp_path):
    model = tiny_opt()
    dense = write_checkpoints(model, tmp_path)
    K.load_shiftaddllm_weight_with_kernel(model, str(tmp_path), "opt-tiny", WBITS, is_lat=True)
    layers = model.model.decoder.layers
    found = K.find_layers(layers[0], layers=(LutLinear,))
    assert set(found) == {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.out_proj", "fc1", "fc2"}
    for i, layer in enumerate(layers):
        for lname, lin in K.find_layers(layer, layers=(LutLinear,)).items():
            assert lin.binaryWeight.shape == (lin.K // 32, WBITS, lin.N) and lin.alpha_layout == "block"
            assert lin.alpha.shape == (lin.K // 8, WBITS, lin.N // GS) and lin.alpha.dtype == torch.float16
            assert lin.bias is not None and lin.group_size == 128            # OPT keeps its biases
            # kernel layout + block alpha dequantise to the same matrix as the checkpoint (also non-square fc1/fc2)
            w = o.dequant_mode_b(lin.binaryWeight.numpy(), lin.alpha.float().numpy())
            assert np.array_equal(w, dense[(i, lname)].numpy())
    # a file whose name promises 2 bits but holds 3 planes is refused (lut_gemm/kernel.py:152)
    import shutil

    first = next(iter(K.find_layers(tiny_opt().model.decoder.layers[0])))
    shutil.copy(f"{tmp_path}/opt-tiny_0.{first}_{WBITS}bit.pt", f"{tmp_path}/opt-tiny_0.{first}_2bit.pt")
    with pytest.raises(ValueError):
        K.load_shiftaddllm_weight_with_kernel(tiny_opt(), str(tmp_path), "opt-tiny", 2, is_lat=True)


def test_checkpoint_writer_undoes_the_activation_order(tmp_path):
    """With act-order the quantiser sees blocks of 8 input rows in permuted order; the writer puts planes and
    alpha back in model order (quant_methods/shiftaddllm.py:195-201).  Checked against the oracle's packer."""
    gen = torch.Generator().manual_seed(11)
    k_in, n_out = 64, 96
    planes = torch.randint(0, 2, (k_in, n_out // GS, GS, WBITS), generator=gen, dtype=torch.int8) * 2 - 1
    alpha = torch.rand(k_in // 8, n_out // GS, WBITS, generator=gen)
    perm = torch.randperm(k_in // 8, generator=gen)
    invperm = torch.argsort(perm)
    permuted_planes = planes.reshape(k_in // 8, 8, -1)[perm].reshape(planes.shape)     # what the quantiser produced
    path = K.save_lat_checkpoint(permuted_planes, alpha[perm], str(tmp_path), "m", "0.fc1", invperm=invperm)
    ckpt = torch.load(path)
    assert np.array_equal(ckpt["bWeight"].numpy(), o.pack_binary_weight(planes.numpy()))
    assert torch.equal(ckpt["alpha"], alpha)
    with pytest.raises(ValueError):
        K.save_lat_checkpoint(planes, alpha, str(tmp_path), "m", "0.fc1", wbits=2)
    with pytest.raises(ValueError):
        K.save_lat_checkpoint(planes, alpha[:-1], str(tmp_path), "m", "0.fc1")


@pytest.mark.gpu
def test_checkpoint_writer_packs_on_the_gpu(tmp_path):
    gen = torch.Generator().manual_seed(12)
    planes = torch.randint(0, 2, (256, 16, GS, WBITS), generator=gen, dtype=torch.int8) * 2 - 1
    alpha = torch.rand(32, 16, WBITS, generator=gen)
    a = torch.load(K.save_lat_checkpoint(planes, alpha, str(tmp_path), "cpu", "0.q"))
    b = torch.load(K.save_lat_checkpoint(planes.cuda(), alpha.cuda(), str(tmp_path), "gpu", "0.q"))
    assert torch.equal(a["bWeight"], b["bWeight"]) and torch.equal(a["alpha"], b["alpha"]) and not b["bWeight"].is_cuda


@pytest.mark.gpu
def test_kernel_path_matches_dense_path_on_gpu(tmp_path):
    """Whole-model check of the drop-in: logits with LutLinear layers (block kernel) vs logits with
    the dequantised dense weights, same checkpoint files."""
    sim, ker = tiny_opt(), tiny_opt()
    write_checkpoints(sim, tmp_path)
    K.load_shiftaddllm_weight(sim, str(tmp_path), "opt-tiny", WBITS, is_lat=True)
    K.load_shiftaddllm_weight_with_kernel(ker, str(tmp_path), "opt-tiny", WBITS, is_lat=True)
    sim, ker = sim.cuda(), ker.cuda()
    for m in ker.modules():
        if isinstance(m, LutLinear) and m.bias is not None:
            m.bias = m.bias.cuda()
    ids = torch.randint(0, 512, (1, 12), generator=torch.Generator().manual_seed(3)).cuda()
    with torch.no_grad():
        ref = sim(ids).logits.float()
        got = ker(ids).logits.float()
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < 2e-2, err

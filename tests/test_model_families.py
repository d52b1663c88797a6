"""`make_lut` on the model families the reference drives besides OPT (model/llama.py:93-98,
model/mistral.py, model/gemma.py, model/bloom.py; linear names as in quant_methods/quant_model_bcq.py:5): tiny
randomly initialised HuggingFace models (no network needed), every decoder-block linear swapped for a
LutLinear holding synthetic BCQ weights, logits compared on the GPU with the same model carrying the
dequantised dense weights — the whole-model form of the drop-in, as tests/test_checkpoint_loaders.py does
for OPT."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import bcq_oracle as o
from shiftaddllm_b200 import kernel as K
from shiftaddllm_b200.quant import LutLinear, make_lut

transformers = pytest.importorskip("transformers")
WBITS, G = 3, 128   # hidden 256 / ffn 512 with groups of 128: shapes the TMA-ring kernel takes


def tiny(family):
    torch.manual_seed(0)
    common = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, vocab_size=320,
                  max_position_embeddings=64)
    if family == "llama":
        return transformers.LlamaForCausalLM(transformers.LlamaConfig(num_key_value_heads=2, **common))
    if family == "mistral":
        return transformers.MistralForCausalLM(transformers.MistralConfig(num_key_value_heads=2, sliding_window=32, **common))
    if family == "gemma":
        return transformers.GemmaForCausalLM(transformers.GemmaConfig(num_key_value_heads=1, head_dim=64, **common))
    if family == "bloom":
        return transformers.BloomForCausalLM(transformers.BloomConfig(hidden_size=256, n_layer=2, n_head=4, vocab_size=320))
    raise ValueError(family)


EXPECTED = {
    "llama": {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj",
              "mlp.down_proj"},
    "bloom": {"self_attention.query_key_value", "self_attention.dense", "mlp.dense_h_to_4h", "mlp.dense_4h_to_h"},
}
EXPECTED["mistral"] = EXPECTED["gemma"] = EXPECTED["llama"]


def quantise_in_place(model, seed=0):
    """Gives every decoder-block linear synthetic BCQ weights: returns {(layer, name): (bw, alpha)} in kernel
    layout and writes the dequantised matrix (oracle) into the dense layer."""
    gen = torch.Generator().manual_seed(seed)
    packed = {}
    for i, layer in enumerate(K._decoder_layers(model)):
        for name, lin in K.find_layers(layer).items():
            k, n = lin.in_features, lin.out_features
            bw = torch.randint(-2 ** 31, 2 ** 31, (k // 32, WBITS, n), generator=gen, dtype=torch.int64).to(torch.int32)
            alpha = torch.exp2(-torch.randint(4, 9, (k // G, WBITS, n), generator=gen).float()).half()
            w = o.dequant_mode_a(bw.numpy(), alpha.numpy())                   # [N, K] fp32
            lin.weight.data = torch.from_numpy(w).to(lin.weight.dtype)
            packed[(i, name)] = (bw, alpha)
    return packed


@pytest.mark.parametrize("family", ["llama", "mistral", "gemma", "bloom"])
def test_make_lut_swaps_the_named_linears(family):
    model = tiny(family)
    layers = K._decoder_layers(model)
    names = K.find_layers(layers[0])
    assert set(names) == EXPECTED[family]
    make_lut(layers, K.find_layers(layers), wbit=WBITS, group_size=G)
    for layer in layers:
        found = K.find_layers(layer, layers=(LutLinear,))
        assert set(found) == EXPECTED[family] and not K.find_layers(layer)     # no nn.Linear left in the block
        for lin in found.values():
            assert lin.binaryWeight.shape == (lin.K // 32, WBITS, lin.N) and lin.group_size == G
    assert isinstance(model.lm_head, nn.Linear)                                # outside the decoder blocks: untouched


@pytest.mark.gpu
@pytest.mark.parametrize("family", ["llama", "mistral", "gemma", "bloom"])
def test_logits_with_lutlinear_match_the_dense_model(family):
    dense = tiny(family).half().eval()
    packed = quantise_in_place(dense)
    lut = tiny(family).half().eval()
    lut.load_state_dict(dense.state_dict())
    layers = K._decoder_layers(lut)
    make_lut(layers, K.find_layers(layers), wbit=WBITS, group_size=G)
    for i, layer in enumerate(layers):
        for name, lin in K.find_layers(layer, layers=(LutLinear,)).items():
            bw, alpha = packed[(i, name)]
            lin.binaryWeight = bw.clone()
            lin.set_row_alpha(alpha)
    dense, lut = dense.cuda(), lut.cuda()
    for m in lut.modules():
        if isinstance(m, LutLinear) and m.bias is not None:
            m.bias = nn.Parameter(m.bias.detach().cuda(), requires_grad=False)
    ids = torch.randint(0, 320, (1, 10), generator=torch.Generator().manual_seed(3)).cuda()
    with torch.no_grad():
        ref = dense(ids).logits.float()
        got = lut(ids).logits.float()                  # a 10-token prompt: LutLinear runs the small-batch kernel (M = 10)
        one = lut(ids[:, :1]).logits.float()           # and the single-token call of the reference's forward
        ref_one = dense(ids[:, :1]).logits.float()
    assert float((got - ref).abs().max() / ref.abs().max()) < 2e-2
    assert float((one - ref_one).abs().max() / ref_one.abs().max()) < 2e-2

"""Quantisation configs, loaders and linear methods on CPU (reference fixtures:
pymllm/tests/test_compressed_tensors_config.py, test_compressed_tensors_runtime.py, test_linear_merged.py)."""
import pytest
import torch

from mllm_b200.layers import Linear, MergedLinear
from mllm_b200.ops import reference as ref
from mllm_b200.quantization import get_quantization_config, list_quantization_methods
from mllm_b200.quantization.methods.awq import pack_awq, pack_rows_natural, unpack_awq


def _ct(fmt="pack-quantized", bits=4, group=32, acts=None, ignore=("lm_head",), strategy="group"):
    return {
        "quant_method": "compressed-tensors", "format": fmt, "ignore": list(ignore),
        "config_groups": {"group_0": {"targets": ["Linear"], "weights": {
            "num_bits": bits, "group_size": group, "strategy": strategy, "symmetric": True, "dynamic": False,
            "actorder": None, "type": "int"}, "input_activations": acts}},
    }


W8A8_ACTS = {"num_bits": 8, "strategy": "token", "symmetric": True, "dynamic": True, "type": "int"}


def test_registry():
    assert {"compressed-tensors", "awq_marlin", "awq"} <= set(list_quantization_methods())
    with pytest.raises(ValueError):
        get_quantization_config("nope")


def test_ct_config_parse_and_ignore():
    cfg = get_quantization_config("compressed-tensors").from_config(
        _ct(ignore=["lm_head", "model.language_model.layers.0.linear_attn.out_proj", "re:.*visual.*"]))
    assert cfg.weight_bits == 4 and cfg.group_size == 32 and cfg.input_bits is None
    assert type(cfg.get_quant_method(None, "lm_head")).__name__ == "UnquantizedLinearMethod"
    assert type(cfg.get_quant_method(None, "model.layers.0.linear_attn.out_proj")).__name__ == "UnquantizedLinearMethod"
    assert type(cfg.get_quant_method(None, "model.visual.blocks.0.attn.qkv")).__name__ == "UnquantizedLinearMethod"
    assert type(cfg.get_quant_method(None, "model.layers.1.self_attn.qkv_proj")).__name__ == "CompressedTensorsW4A16Method"


def test_ct_unsupported_scheme_is_clear():
    cfg = get_quantization_config("compressed-tensors").from_config(_ct(bits=3))
    with pytest.raises(ValueError, match="unsupported scheme"):
        cfg.get_quant_method(None, "x")


def _quantize_w4(w, group):
    n, k = w.shape
    wg = w.reshape(n, k // group, group)
    scale = wg.abs().amax(-1) / 7.0
    q = torch.clamp(torch.round(wg / scale.unsqueeze(-1)), -8, 7) + 8
    return q.reshape(n, k).to(torch.uint8), scale


def test_w4a16_linear_matches_dequant_matmul():
    torch.manual_seed(0)
    cfg = get_quantization_config("compressed-tensors").from_config(_ct(group=32))
    lin = Linear(128, 64, quant_method=cfg.get_quant_method(None, "l"), params_dtype=torch.float32)
    w = torch.randn(64, 128)
    q, scale = _quantize_w4(w, 32)
    lin.weight_packed.weight_loader(lin.weight_packed, pack_rows_natural(q))
    lin.weight_scale.weight_loader(lin.weight_scale, scale)
    lin.quant_method.process_weights_after_loading(lin)
    x = torch.randn(5, 128)
    want = x @ ((q.float() - 8) * scale.repeat_interleave(32, 1)).t()
    torch.testing.assert_close(lin(x), want, atol=1e-4, rtol=1e-4)
    assert lin.weight_shape.tolist() == [64, 128]


def test_w4a16_merged_loader_stacks_shards():
    cfg = get_quantization_config("compressed-tensors").from_config(_ct(group=32))
    m = MergedLinear(64, [32, 16, 16], quant_method=cfg.get_quant_method(None, "qkv"), params_dtype=torch.float32,
                     shard_names=["q", "k", "v"])
    for sid, rows, fill in (("q", 32, 1), ("k", 16, 2), ("v", 16, 3)):
        m.weight_packed.weight_loader(m.weight_packed, torch.full((rows, 8), fill, dtype=torch.int32), sid)
        m.weight_scale.weight_loader(m.weight_scale, torch.full((rows, 2), float(fill)), sid)
        m.weight_shape.weight_loader(m.weight_shape, torch.tensor([rows, 64]), sid)
    assert m.weight_packed[:32].eq(1).all() and m.weight_packed[32:48].eq(2).all() and m.weight_packed[48:].eq(3).all()
    assert m.weight_scale[48:].eq(3).all()


def test_w8a8_linear_matches_int_reference():
    torch.manual_seed(1)
    cfg = get_quantization_config("compressed-tensors").from_config(
        _ct(fmt="int-quantized", bits=8, group=None, acts=W8A8_ACTS, strategy="channel"))
    lin = Linear(256, 48, quant_method=cfg.get_quant_method(None, "l"), params_dtype=torch.float32)
    wq = torch.randint(-127, 128, (48, 256), dtype=torch.int8)
    ws = torch.rand(48, 1) * 0.02
    lin.weight.weight_loader(lin.weight, wq)
    lin.weight_scale.weight_loader(lin.weight_scale, ws)
    lin.quant_method.process_weights_after_loading(lin)
    assert lin.weight_scale.shape == (48,) and lin.weight_scale.dtype == torch.float32
    x = torch.randn(7, 256)
    xq, xs = ref.per_token_quant_int8(x)
    want = (xq.float() @ wq.float().t()) * xs * ws.reshape(1, -1)
    torch.testing.assert_close(lin(x), want, atol=1e-4, rtol=1e-4)
    # error of the whole scheme against the float product stays at the int8 level
    full = x @ (wq.float() * ws).t()
    assert ((lin(x) - full).norm() / full.norm()) < 0.02


def test_awq_pack_roundtrip_and_linear():
    torch.manual_seed(2)
    vals = torch.randint(0, 16, (6, 32), dtype=torch.uint8)
    assert torch.equal(unpack_awq(pack_awq(vals)), vals)
    # word layout: logical column 1 sits in nibble position 4
    one = torch.zeros(1, 8, dtype=torch.uint8)
    one[0, 1] = 0xF
    assert int(pack_awq(one)[0, 0]) == 0xF << 16

    K, N, g = 128, 64, 32
    cfg = get_quantization_config("awq").from_config({"w_bit": 4, "q_group_size": g, "zero_point": True})
    lin = Linear(K, N, quant_method=cfg.get_quant_method(None, "l"), params_dtype=torch.float32)
    q = torch.randint(0, 16, (K, N), dtype=torch.uint8)
    z = torch.randint(0, 16, (K // g, N), dtype=torch.uint8)
    s = torch.rand(K // g, N) * 0.1
    lin.qweight.weight_loader(lin.qweight, pack_awq(q))
    lin.qzeros.weight_loader(lin.qzeros, pack_awq(z))
    lin.scales.weight_loader(lin.scales, s)
    lin.quant_method.process_weights_after_loading(lin)
    assert lin.weight_packed.shape == (N, K // 8) and lin.weight_zeros.shape == (N, K // g)
    w = (q.float() - z.float().repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)  # [K, N]
    x = torch.randn(3, K)
    torch.testing.assert_close(lin(x), x @ w, atol=1e-4, rtol=1e-4)


def test_awq_config_keys():
    cls = get_quantization_config("awq_marlin")
    assert cls.from_config({"bits": 4, "group_size": 128, "zero_point": True}).group_size == 128
    with pytest.raises(ValueError):
        cls.from_config({"bits": 8, "group_size": 128})
    assert cls.get_config_filenames() == ["quant_config.json", "quantize_config.json"]

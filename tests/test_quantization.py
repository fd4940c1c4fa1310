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


def test_gptq_layout_linear_and_tensor_parallel_shards():
    """GPTQ tensors (qweight packed along K, qzeros packed along N and stored minus one) -> the K-major
    4-bit layout; the linear equals the dequantised matmul; column- and row-parallel shards of the packed
    tensors give the matching slices of the full result."""
    from mllm_b200.layers.linear import ColumnParallelLinear, RowParallelLinear
    from mllm_b200.quantization.methods.gptq import pack_words, unpack_words

    torch.manual_seed(5)
    vals = torch.randint(0, 16, (16, 24), dtype=torch.uint8)
    assert torch.equal(unpack_words(pack_words(vals, 0), 0), vals) and torch.equal(unpack_words(pack_words(vals, 1), 1), vals)
    col = torch.zeros(8, 1, dtype=torch.uint8)
    col[1, 0] = 0xF                                       # input channel 1 sits in the second nibble of the word
    assert int(pack_words(col, 0)[0, 0]) == 0xF << 4

    K, N, g = 128, 64, 32
    cfg = get_quantization_config("gptq").from_config({"bits": 4, "group_size": g, "sym": False, "desc_act": False})
    q = torch.randint(0, 16, (K, N), dtype=torch.uint8)
    z = torch.randint(1, 16, (K // g, N), dtype=torch.uint8)
    s = torch.rand(K // g, N) * 0.1
    w = (q.float() - z.float().repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)       # [K, N]
    tensors = {"qweight": pack_words(q, 0), "qzeros": pack_words(z - 1, 1), "scales": s, "g_idx": torch.arange(K, dtype=torch.int32) // g}

    def build(cls, *a, **kw):
        lin = cls(*a, quant_method=cfg.get_quant_method(None, "l"), params_dtype=torch.float32, **kw)
        for name, t in tensors.items():
            p = getattr(lin, name)
            p.weight_loader(p, t)
        lin.quant_method.process_weights_after_loading(lin)
        return lin

    lin = build(Linear, K, N)
    assert lin.weight_packed.shape == (N, K // 8) and lin.weight_zeros.shape == (N, K // g) and not hasattr(lin, "g_idx")
    x = torch.randn(3, K)
    torch.testing.assert_close(lin(x), x @ w, atol=1e-4, rtol=1e-4)
    # the classic format's "zero - 1" against the v2 format's plain zero
    v2 = get_quantization_config("gptq").from_config({"bits": 4, "group_size": g, "checkpoint_format": "gptq_v2"})
    assert v2.get_quant_method(None, "l").zero_offset == 0 and cfg.get_quant_method(None, "l").zero_offset == 1
    with pytest.raises(ValueError):
        get_quantization_config("gptq").from_config({"bits": 8, "group_size": g})
    # activation order: channel k belongs to group g_idx[k]; rows sorted by group at load, x permuted at run time
    act = get_quantization_config("gptq").from_config({"bits": 4, "group_size": g, "sym": False, "desc_act": True})
    gi = (torch.arange(K) // g)[torch.randperm(K)].to(torch.int32)
    w_act = (q.float() - z.float()[gi.long()]) * s[gi.long()]                            # [K, N]
    lin_a = Linear(K, N, quant_method=act.get_quant_method(None, "l"), params_dtype=torch.float32)
    for name, t in dict(tensors, g_idx=gi).items():
        p = getattr(lin_a, name)
        p.weight_loader(p, t)
    lin_a.quant_method.process_weights_after_loading(lin_a)
    assert lin_a.act_perm is not None
    torch.testing.assert_close(lin_a(x), x @ w_act, atol=1e-4, rtol=1e-4)

    # shards as a 2-rank job would load them
    import mllm_b200.parallel.state as pstate

    class FakeTP:
        def __init__(self, r):
            self.world_size, self.rank_in_group = 2, r

    saved = pstate._TP
    try:
        for r in range(2):
            pstate._TP = FakeTP(r)
            colp = build(ColumnParallelLinear, K, N)
            torch.testing.assert_close(colp(x), (x @ w)[:, r * N // 2:(r + 1) * N // 2], atol=1e-4, rtol=1e-4)
            rowp = build(RowParallelLinear, K, N, reduce_results=False)
            xs = x[:, r * K // 2:(r + 1) * K // 2]
            torch.testing.assert_close(rowp.quant_method.apply(rowp, xs), xs @ w[r * K // 2:(r + 1) * K // 2], atol=1e-4, rtol=1e-4)
    finally:
        pstate._TP = saved


def test_gptq_checkpoint_directory_end_to_end(tmp_path):
    """A GPTQ checkpoint directory (config.json with quantization_config + safetensors with qweight / qzeros /
    scales / g_idx per projection) served by the model runner gives the logits of the dense model built from
    the dequantised weights."""
    import json

    from safetensors.torch import save_file

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.models.presets import get_preset, preset_to_config_json
    from mllm_b200.quantization.methods.gptq import pack_words

    cfg_json = dict(preset_to_config_json("qwen3-tiny"), tie_word_embeddings=False,
                    quantization_config={"quant_method": "gptq", "bits": 4, "group_size": 32, "sym": True, "desc_act": False})
    cfg = get_preset("qwen3-tiny", tie_word_embeddings=False)
    g = torch.Generator().manual_seed(0)
    sd_q, sd_d = {}, {}
    H, D, I, V = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size

    def dense(name, t):
        sd_q[name] = sd_d[name] = t

    def quant(prefix, n, k):
        q = torch.randint(0, 16, (k, n), generator=g, dtype=torch.uint8)
        s = torch.rand(k // 32, n, generator=g) * 0.02
        z = torch.randint(1, 16, (k // 32, n), generator=g, dtype=torch.uint8)
        sd_q[prefix + ".qweight"], sd_q[prefix + ".qzeros"], sd_q[prefix + ".scales"] = pack_words(q, 0), pack_words(z - 1, 1), s
        sd_q[prefix + ".g_idx"] = torch.arange(k, dtype=torch.int32) // 32
        sd_d[prefix + ".weight"] = ((q.float() - z.float().repeat_interleave(32, 0)) * s.repeat_interleave(32, 0)).t().contiguous()

    dense("model.embed_tokens.weight", torch.randn(V, H, generator=g) * 0.05)
    dense("lm_head.weight", torch.randn(V, H, generator=g) * 0.05)
    dense("model.norm.weight", torch.ones(H))
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        for nm, n, k in (("self_attn.q_proj", hq * D, H), ("self_attn.k_proj", hkv * D, H), ("self_attn.v_proj", hkv * D, H),
                         ("self_attn.o_proj", H, hq * D), ("mlp.gate_proj", I, H), ("mlp.up_proj", I, H), ("mlp.down_proj", H, I)):
            quant(p + nm, n, k)
        for nm, d in (("self_attn.q_norm.weight", D), ("self_attn.k_norm.weight", D), ("input_layernorm.weight", H),
                      ("post_attention_layernorm.weight", H)):
            dense(p + nm, torch.ones(d) + torch.randn(d, generator=g) * 0.05)
    logits = []
    for name, sd, extra in (("gptq", sd_q, cfg_json), ("dense", sd_d, {k: v for k, v in cfg_json.items() if k != "quantization_config"})):
        d = tmp_path / name
        d.mkdir()
        (d / "config.json").write_text(json.dumps(extra))
        save_file({k: v.contiguous() for k, v in sd.items()}, str(d / "model.safetensors"))
        mr = ModelRunner(ServerConfig(model_path=str(d), dtype="float32", max_running_requests=2, max_total_tokens=256), device="cpu")
        mr.initialize()
        if name == "gptq":
            assert type(mr.quant_config).__name__ == "GPTQConfig"
            assert mr.model.model.layers[0].self_attn.qkv_proj.weight_packed.shape == ((hq + 2 * hkv) * D, H // 8)
        ids = torch.arange(9) * 7 % V
        slots = mr.req_to_token_pool.alloc(1)
        loc = mr.token_to_kv_pool_allocator.alloc(9)
        mr.req_to_token_pool.req_to_token[slots[0], :9] = loc.int()
        lens = torch.tensor([9])
        fb = mr.prepare_forward_batch_extend(ids, torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)
        logits.append(mr.forward(fb).next_token_logits)
    torch.testing.assert_close(logits[0], logits[1], atol=2e-4, rtol=2e-4)


def test_fp8_block_and_per_tensor_weights_expand_to_the_dequantised_model():
    from mllm_b200.layers.linear import MergedLinear

    torch.manual_seed(9)
    K, N, b = 256, 384, 128
    cfg = get_quantization_config("fp8").from_config({"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [b, b]})
    lin = Linear(K, N, quant_method=cfg.get_quant_method(None, "l"), params_dtype=torch.float32)
    w8 = (torch.randn(N, K) * 2).to(torch.float8_e4m3fn)
    sc = torch.rand(N // b, K // b) * 0.1 + 0.01
    lin.weight.weight_loader(lin.weight, w8)
    lin.weight_scale_inv.weight_loader(lin.weight_scale_inv, sc)
    lin.quant_method.process_weights_after_loading(lin)
    want = w8.float() * sc.repeat_interleave(b, 0).repeat_interleave(b, 1)
    assert lin.weight.dtype == torch.float32 and not hasattr(lin, "weight_scale_inv")
    x = torch.randn(3, K)
    torch.testing.assert_close(lin(x), x @ want.t(), atol=1e-4, rtol=1e-4)
    # fused q/k/v with block scales: every shard lands at its block offset
    m = MergedLinear(K, [256, 128, 128], quant_method=cfg.get_quant_method(None, "qkv"), params_dtype=torch.float32,
                     shard_names=["q", "k", "v"])
    parts = []
    for sid, n in (("q", 256), ("k", 128), ("v", 128)):
        w = (torch.randn(n, K) * 2).to(torch.float8_e4m3fn)
        s = torch.rand(n // b, K // b) * 0.1 + 0.01
        m.weight.weight_loader(m.weight, w, sid)
        m.weight_scale_inv.weight_loader(m.weight_scale_inv, s, sid)
        parts.append(w.float() * s.repeat_interleave(b, 0).repeat_interleave(b, 1))
    m.quant_method.process_weights_after_loading(m)
    torch.testing.assert_close(m(x), x @ torch.cat(parts, 0).t(), atol=1e-4, rtol=1e-4)
    # per-tensor scales
    cfg_t = get_quantization_config("fp8").from_config({"quant_method": "fp8"})
    lin_t = Linear(K, N, quant_method=cfg_t.get_quant_method(None, "l"), params_dtype=torch.float32)
    lin_t.weight.weight_loader(lin_t.weight, w8)
    lin_t.weight_scale.weight_loader(lin_t.weight_scale, torch.tensor(0.25))
    lin_t.quant_method.process_weights_after_loading(lin_t)
    torch.testing.assert_close(lin_t(x), x @ (w8.float() * 0.25).t(), atol=1e-4, rtol=1e-4)
    assert type(cfg.get_quant_method(None, "lm_head")).__name__ == "UnquantizedLinearMethod"
    with pytest.raises(ValueError):
        get_quantization_config("fp8").from_config({"fmt": "e5m2"})


def test_ct_w8a16_channel_group_and_packed_expand_to_the_dequantised_weights():
    torch.manual_seed(11)
    K, N = 128, 48
    x = torch.randn(3, K)
    q = torch.randint(-127, 128, (N, K), dtype=torch.int8)
    # per channel, int-quantized
    cfg = get_quantization_config("compressed-tensors").from_config(_ct(fmt="int-quantized", bits=8, group=None, strategy="channel"))
    lin = Linear(K, N, quant_method=cfg.get_quant_method(None, "l"), params_dtype=torch.float32)
    assert type(lin.quant_method).__name__ == "CompressedTensorsW8A16Method"
    s = torch.rand(N, 1) * 0.01 + 0.001
    lin.weight.weight_loader(lin.weight, q)
    lin.weight_scale.weight_loader(lin.weight_scale, s)
    lin.quant_method.process_weights_after_loading(lin)
    torch.testing.assert_close(lin(x), x @ (q.float() * s).t(), atol=1e-4, rtol=1e-4)
    # per group of 32, pack-quantized (four offset-binary bytes per word)
    cfg_g = get_quantization_config("compressed-tensors").from_config(_ct(fmt="pack-quantized", bits=8, group=32))
    lin_g = Linear(K, N, quant_method=cfg_g.get_quant_method(None, "l"), params_dtype=torch.float32)
    sg = torch.rand(N, K // 32) * 0.01 + 0.001
    u = (q.to(torch.int64) + 128).reshape(N, K // 4, 4)
    words = (u[..., 0] | (u[..., 1] << 8) | (u[..., 2] << 16) | (u[..., 3] << 24))
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    lin_g.weight_packed.weight_loader(lin_g.weight_packed, words)
    lin_g.weight_scale.weight_loader(lin_g.weight_scale, sg)
    lin_g.quant_method.process_weights_after_loading(lin_g)
    assert not hasattr(lin_g, "weight_packed") and lin_g.weight.shape == (N, K)
    torch.testing.assert_close(lin_g(x), x @ (q.float() * sg.repeat_interleave(32, 1)).t(), atol=1e-4, rtol=1e-4)

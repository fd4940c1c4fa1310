"""Qwen3-MoE on CPU: router/expert semantics against a direct restatement of the reference's C++
MoE (softmax -> top-k -> renorm -> per-expert SwiGLU -> weighted sum) and against HF transformers."""
import types

import pytest
import torch
import torch.nn.functional as F

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner
from mllm_b200.models.presets import get_preset
from mllm_b200.models.qwen3_moe import is_sparse_layer
from mllm_b200.ops import reference as ref


def test_sparse_layer_rule():
    cfg = types.SimpleNamespace(num_experts=8, decoder_sparse_step=2, mlp_only_layers=[3])
    assert [is_sparse_layer(cfg, i) for i in range(6)] == [False, True, False, False, False, True]
    assert not is_sparse_layer(types.SimpleNamespace(num_experts=0), 0)


def test_router_and_experts_match_reference_semantics():
    torch.manual_seed(0)
    T, H, E, I, k = 9, 32, 6, 16, 2
    x, wg = torch.randn(T, H), torch.randn(E, H)
    w13, w2 = torch.randn(E, 2 * I, H) * 0.2, torch.randn(E, H, I) * 0.2
    tw, ti = ref.moe_router_topk(x, wg, k, True)
    scores = torch.softmax(x @ wg.t(), -1)
    assert torch.equal(ti.long(), scores.topk(k, -1).indices)
    torch.testing.assert_close(tw.sum(-1), torch.ones(T))
    got = ref.moe_experts(x, w13, w2, tw, ti)
    want = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ti[t, j])
            g, u = x[t] @ w13[e, :I].t(), x[t] @ w13[e, I:].t()
            want[t] += tw[t, j] * ((F.silu(g) * u) @ w2[e].t())
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)
    # expert-parallel split: two halves of the experts sum to the whole
    a = ref.moe_experts(x, w13[:3], w2[:3], tw, ti, expert_offset=0)
    b = ref.moe_experts(x, w13[3:], w2[3:], tw, ti, expert_offset=3)
    torch.testing.assert_close(a + b, got, atol=1e-5, rtol=1e-5)


def test_matches_hf_qwen3_moe():
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=2,
                num_attention_heads=2, num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
                tie_word_embeddings=False, max_position_embeddings=256, attention_bias=False, num_experts=4,
                num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])
    try:
        hf = tr.Qwen3MoeForCausalLM(tr.Qwen3MoeConfig(**cfgd)).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3-MoE unavailable: {e}")
    ns = types.SimpleNamespace(architectures=["Qwen3MoeForCausalLM"], **cfgd)
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    sd = hf.state_dict()
    # newer transformers keep the experts fused in two 3-D tensors: the loader splits them
    mr.model.load_weights(sd.items())
    ids = torch.randint(0, 300, (1, 10))
    slots = mr.req_to_token_pool.alloc(1)
    loc = mr.token_to_kv_pool_allocator.alloc(10)
    mr.req_to_token_pool.req_to_token[slots[0], :10] = loc.int()
    lens = torch.tensor([10])
    fb = mr.prepare_forward_batch_extend(ids.reshape(-1), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(got, want, atol=3e-4, rtol=3e-4)


def test_moe_preset_runs():
    mr = ModelRunner(ServerConfig(model_path="preset:qwen3-moe-tiny", dtype="float32", max_running_requests=2,
                                  max_total_tokens=256), device="cpu")
    mr.initialize()
    assert type(mr.model).__name__ == "Qwen3MoeForCausalLM"
    assert sum(1 for n, _ in mr.model.named_parameters() if n.endswith("block.w13")) == 2


def _compare_moe_family(arch, hf, cfgd, rename=None):
    ns = types.SimpleNamespace(architectures=[arch], head_dim=16, **cfgd)
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    sd = hf.state_dict()
    if rename is not None:
        sd = rename(sd)
    loaded = mr.model.load_weights(sd.items())
    missing = set(dict(mr.model.named_parameters())) - loaded
    assert not missing, missing
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
        if hasattr(m, "swiglu_block") and hasattr(m, "w13"):
            m.swiglu_block = 0
    mr.model.post_load()
    torch.manual_seed(0)
    ids = torch.randint(0, cfgd["vocab_size"], (1, 11))
    slots = mr.req_to_token_pool.alloc(1)
    loc = mr.token_to_kv_pool_allocator.alloc(11)
    mr.req_to_token_pool.req_to_token[slots[0], :11] = loc.int()
    lens = torch.tensor([11])
    fb = mr.prepare_forward_batch_extend(ids.reshape(-1), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(got, want, atol=1e-3, rtol=1e-3)


def _spread(hf):
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("mlp.gate.weight") or n.endswith("shared_expert_gate.weight"):
                p.copy_(torch.randn_like(p))
            if "experts" in n:
                p.copy_(torch.randn_like(p) * 0.05)
            if n.endswith(".bias"):
                p.copy_(torch.randn_like(p) * 0.05)


def test_qwen2_moe_matches_hf():
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32, shared_expert_intermediate_size=48,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, num_experts=4, num_experts_per_tok=2,
                norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[1], rms_norm_eps=1e-6, rope_theta=10000.0,
                tie_word_embeddings=False, max_position_embeddings=256, use_sliding_window=False)
    try:
        hf = tr.Qwen2MoeForCausalLM(tr.Qwen2MoeConfig(**cfgd)).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen2-MoE unavailable: {e}")
    _spread(hf)
    _compare_moe_family("Qwen2MoeForCausalLM", hf, cfgd)


def test_mixtral_matches_hf_with_hub_style_names():
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2, rms_norm_eps=1e-5, rope_theta=10000.0,
                tie_word_embeddings=False, max_position_embeddings=256, sliding_window=None)
    try:
        hf = tr.MixtralForCausalLM(tr.MixtralConfig(**cfgd)).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Mixtral unavailable: {e}")
    _spread(hf)

    def hub_names(sd):
        """The layout of the published checkpoints: block_sparse_moe.gate / experts.N.w1 (gate), w3 (up), w2 (down)."""
        out = {}
        for k, v in sd.items():
            if k.endswith("mlp.experts.gate_up_proj"):
                base = k[: -len("mlp.experts.gate_up_proj")] + "block_sparse_moe.experts."
                for e in range(v.shape[0]):
                    out[f"{base}{e}.w1.weight"], out[f"{base}{e}.w3.weight"] = v[e, :96], v[e, 96:]
            elif k.endswith("mlp.experts.down_proj"):
                base = k[: -len("mlp.experts.down_proj")] + "block_sparse_moe.experts."
                for e in range(v.shape[0]):
                    out[f"{base}{e}.w2.weight"] = v[e]
            else:
                out[k.replace(".mlp.gate.", ".block_sparse_moe.gate.")] = v
        return out

    _compare_moe_family("MixtralForCausalLM", hf, cfgd, rename=hub_names)
    _compare_moe_family("MixtralForCausalLM", hf, cfgd)          # and the fused in-memory layout


def test_gptq_quantised_moe_checkpoint_loads_like_its_dequantised_twin(tmp_path):
    """A GPTQ checkpoint of the tiny MoE model — attention projections served by the 4-bit linear method,
    expert projections dequantised at load — gives the logits of the dense model built from the same
    dequantised weights."""
    import json

    from safetensors.torch import save_file

    from mllm_b200.models.presets import get_preset, preset_to_config_json
    from mllm_b200.quantization.methods.gptq import pack_words

    cfg = get_preset("qwen3-moe-tiny", tie_word_embeddings=False)
    cfg_json = dict(preset_to_config_json("qwen3-moe-tiny"), tie_word_embeddings=False,
                    quantization_config={"quant_method": "gptq", "bits": 4, "group_size": 32, "sym": True, "desc_act": False})
    g = torch.Generator().manual_seed(1)
    H, D, V, E, Im = cfg.hidden_size, cfg.head_dim, cfg.vocab_size, cfg.num_experts, cfg.moe_intermediate_size
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    sd_q, sd_d = {}, {}

    def dense(name, t):
        sd_q[name] = sd_d[name] = t

    def quant(prefix, n, k):
        q = torch.randint(0, 16, (k, n), generator=g, dtype=torch.uint8)
        s = torch.rand(k // 32, n, generator=g) * 0.02
        z = torch.full((k // 32, n), 8, dtype=torch.uint8)
        sd_q[prefix + ".qweight"], sd_q[prefix + ".qzeros"], sd_q[prefix + ".scales"] = pack_words(q, 0), pack_words(z - 1, 1), s
        sd_q[prefix + ".g_idx"] = torch.arange(k, dtype=torch.int32) // 32
        sd_d[prefix + ".weight"] = ((q.float() - 8) * s.repeat_interleave(32, 0)).t().contiguous()

    dense("model.embed_tokens.weight", torch.randn(V, H, generator=g) * 0.05)
    dense("lm_head.weight", torch.randn(V, H, generator=g) * 0.05)
    dense("model.norm.weight", torch.ones(H))
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        for nm, n, k in (("self_attn.q_proj", hq * D, H), ("self_attn.k_proj", hkv * D, H), ("self_attn.v_proj", hkv * D, H),
                         ("self_attn.o_proj", H, hq * D)):
            quant(p + nm, n, k)
        dense(p + "mlp.gate.weight", torch.randn(E, H, generator=g))
        for e in range(E):
            quant(p + f"mlp.experts.{e}.gate_proj", Im, H)
            quant(p + f"mlp.experts.{e}.up_proj", Im, H)
            quant(p + f"mlp.experts.{e}.down_proj", H, Im)
        for nm, d in (("self_attn.q_norm.weight", D), ("self_attn.k_norm.weight", D), ("input_layernorm.weight", H),
                      ("post_attention_layernorm.weight", H)):
            dense(p + nm, torch.ones(d))
    logits = []
    for name, sd, cj in (("gptq", sd_q, cfg_json), ("dense", sd_d, {k: v for k, v in cfg_json.items() if k != "quantization_config"})):
        d = tmp_path / name
        d.mkdir()
        (d / "config.json").write_text(json.dumps(cj))
        save_file({k: v.contiguous() for k, v in sd.items()}, str(d / "model.safetensors"))
        mr = ModelRunner(ServerConfig(model_path=str(d), dtype="float32", max_running_requests=2, max_total_tokens=256), device="cpu")
        mr.initialize()
        ids = torch.arange(10) * 11 % V
        slots = mr.req_to_token_pool.alloc(1)
        loc = mr.token_to_kv_pool_allocator.alloc(10)
        mr.req_to_token_pool.req_to_token[slots[0], :10] = loc.int()
        lens = torch.tensor([10])
        fb = mr.prepare_forward_batch_extend(ids, torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)
        logits.append(mr.forward(fb).next_token_logits)
    torch.testing.assert_close(logits[0], logits[1], atol=3e-4, rtol=3e-4)

"""Llama-family and Qwen2-family decoders against HF transformers on CPU (prefill in two chunks, then
decode): no q/k norm, optional q/k/v biases, ``llama3`` / ``linear`` rotary rescaling."""

import types

import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner


def _run_and_compare(hf, ns, vocab):
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=512),
                     hf_config=ns, device="cpu")
    mr.initialize()
    loaded = mr.model.load_weights(hf.state_dict().items())
    missing = set(dict(mr.model.named_parameters())) - loaded
    assert not missing, missing
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    torch.manual_seed(0)
    ids = torch.randint(0, vocab, (1, 40))
    slots = mr.req_to_token_pool.alloc(1)
    sl = torch.tensor(slots)
    loc = mr.token_to_kv_pool_allocator.alloc(40)
    mr.req_to_token_pool.req_to_token[slots[0], :40] = loc.int()
    fb = mr.prepare_forward_batch_extend(ids[0, :23], sl, torch.tensor([23]), torch.tensor([23]), torch.tensor([0]), loc[:23])
    mr.forward(fb)
    fb = mr.prepare_forward_batch_extend(ids[0, 23:], sl, torch.tensor([40]), torch.tensor([17]), torch.tensor([23]), loc[23:])
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)
    cur, seq = 40, ids
    for _ in range(2):
        nxt = got.argmax(-1)
        loc1 = mr.token_to_kv_pool_allocator.alloc(1)
        mr.req_to_token_pool.req_to_token[slots[0], cur] = loc1.int()
        cur += 1
        got = mr.forward(mr.prepare_forward_batch_decode(nxt, sl, torch.tensor([cur]), loc1)).next_token_logits
        seq = torch.cat([seq, nxt[:, None]], 1)
        with torch.no_grad():
            want = hf(seq).logits[:, -1]
        torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)


@pytest.mark.parametrize("scaling", [None,
                                     dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                          original_max_position_embeddings=16),
                                     dict(rope_type="linear", factor=2.0)])
def test_llama_matches_hf(scaling):
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
                attention_bias=False, mlp_bias=False, hidden_act="silu", rope_theta=10000.0)
    try:
        hf_cfg = tr.LlamaConfig(**cfgd, rope_scaling=dict(scaling) if scaling else None)
        hf = tr.LlamaForCausalLM(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Llama unavailable: {e}")
    ns = types.SimpleNamespace(architectures=["LlamaForCausalLM"], head_dim=16, rope_scaling=scaling, **cfgd)
    _run_and_compare(hf, ns, 320)


def test_qwen2_matches_hf():
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256,
                hidden_act="silu", rope_theta=10000.0, use_sliding_window=False)
    try:
        hf = tr.Qwen2ForCausalLM(tr.Qwen2Config(**cfgd)).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen2 unavailable: {e}")
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("proj.bias"):
                p.copy_(torch.randn_like(p) * 0.1)
    ns = types.SimpleNamespace(architectures=["Qwen2ForCausalLM"], head_dim=16, **cfgd)
    _run_and_compare(hf, ns, 320)


def test_smollm3_matches_hf():
    """Every fourth layer attends without rotary embedding."""
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256,
                attention_bias=False, mlp_bias=False, hidden_act="silu", use_sliding_window=False)
    try:
        hf_cfg = tr.SmolLM3Config(**cfgd, pad_token_id=0, rope_parameters=dict(rope_theta=10000.0, rope_type="default"))
        hf = tr.SmolLM3ForCausalLM(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers SmolLM3 unavailable: {e}")
    assert list(hf_cfg.no_rope_layers) == [1, 1, 1, 0]
    ns = types.SimpleNamespace(architectures=["SmolLM3ForCausalLM"], head_dim=16, rope_theta=10000.0,
                               no_rope_layers=[1, 1, 1, 0], **cfgd)
    _run_and_compare(hf, ns, 320)


def test_unsupported_variants_are_refused():
    from mllm_b200.models import get_model_class

    cfg = types.SimpleNamespace(vocab_size=32, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                                num_key_value_heads=2, rms_norm_eps=1e-6, tie_word_embeddings=True, sliding_window=128)
    with pytest.raises(NotImplementedError):
        get_model_class("MistralForCausalLM")(cfg)
    cfg2 = types.SimpleNamespace(**{**vars(cfg), "sliding_window": None, "rope_scaling": dict(rope_type="yarn", factor=4.0)})
    with pytest.raises(NotImplementedError):
        m = get_model_class("LlamaForCausalLM")(cfg2)
        m.model.layers[0].self_attn.attn._tables(torch.device("cpu"))

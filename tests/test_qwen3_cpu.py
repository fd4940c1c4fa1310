"""The Qwen3 decoder on CPU (fp32 PyTorch statements of the ops) against HF transformers on a tiny
random config, plus loader and residual-carry checks."""
import types

import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner
from mllm_b200.models import get_model_class, supported_architectures
from mllm_b200.models.presets import get_preset


def _runner(preset="qwen3-tiny", **kw):
    sc = ServerConfig(model_path=f"preset:{preset}", dtype="float32", max_running_requests=4, max_total_tokens=2048, **kw)
    mr = ModelRunner(sc, device="cpu")
    mr.initialize()
    return mr


def _prefill(mr, ids_2d):
    B, L = ids_2d.shape
    slots = mr.req_to_token_pool.alloc(B)
    loc = mr.token_to_kv_pool_allocator.alloc(B * L)
    for i, s in enumerate(slots):
        mr.req_to_token_pool.req_to_token[s, :L] = loc[i * L:(i + 1) * L].int()
    lens = torch.full((B,), L)
    fb = mr.prepare_forward_batch_extend(ids_2d.reshape(-1), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)
    return slots, mr.forward(fb).next_token_logits


def _decode(mr, slots, cur_len, ids):
    B = len(slots)
    loc = mr.token_to_kv_pool_allocator.alloc(B)
    for i, s in enumerate(slots):
        mr.req_to_token_pool.req_to_token[s, cur_len] = loc[i].int()
    fb = mr.prepare_forward_batch_decode(ids, torch.tensor(slots), torch.full((B,), cur_len + 1), loc)
    return mr.forward(fb).next_token_logits


def test_registry():
    assert "Qwen3ForCausalLM" in supported_architectures()
    assert get_model_class("Qwen3ForCausalLM").__name__ == "Qwen3ForCausalLM"
    with pytest.raises(ValueError):
        get_model_class("NopeForCausalLM")


def test_matches_hf_transformers_prefill_and_decode():
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False,
                max_position_embeddings=512, attention_bias=False)
    try:
        hf_cfg = tr.Qwen3Config(**cfgd)
        hf = tr.Qwen3ForCausalLM(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3 unavailable: {e}")
    ns = types.SimpleNamespace(architectures=["Qwen3ForCausalLM"], **cfgd)
    sc = ServerConfig(model_path="preset:unused", dtype="float32", max_running_requests=2, max_total_tokens=512)
    mr = ModelRunner(sc, hf_config=ns, device="cpu")
    mr.initialize()
    loaded = mr.model.load_weights(hf.state_dict().items())
    assert len(loaded) == len(dict(mr.model.named_parameters()))
    for m in mr.model.modules():  # re-run the post-load step on the freshly loaded weights
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    torch.manual_seed(0)
    ids = torch.randint(0, 512, (2, 11))
    slots, logits = _prefill(mr, ids)
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(logits, want, atol=2e-4, rtol=2e-4)
    nxt = logits.argmax(-1)
    got2 = _decode(mr, slots, 11, nxt)
    with torch.no_grad():
        want2 = hf(torch.cat([ids, nxt[:, None]], 1)).logits[:, -1]
    torch.testing.assert_close(got2, want2, atol=2e-4, rtol=2e-4)


def test_decode_equals_recomputed_prefill():
    mr = _runner()
    torch.manual_seed(1)
    ids = torch.randint(0, 1024, (1, 9))
    slots, logits = _prefill(mr, ids)
    nxt = logits.argmax(-1)
    dec = _decode(mr, slots, 9, nxt)
    mr2 = _runner()
    _, full = _prefill(mr2, torch.cat([ids, nxt[:, None]], 1))
    torch.testing.assert_close(dec, full, atol=1e-4, rtol=1e-4)


def test_prefix_reuse_equals_full_prefill():
    """Extending after a cached prefix gives the logits of a full prefill."""
    mr = _runner()
    torch.manual_seed(2)
    ids = torch.randint(0, 1024, (1, 12))
    _, want = _prefill(mr, ids)
    mr2 = _runner()
    slots, _ = _prefill(mr2, ids[:, :7])
    loc = mr2.token_to_kv_pool_allocator.alloc(5)
    mr2.req_to_token_pool.req_to_token[slots[0], 7:12] = loc.int()
    fb = mr2.prepare_forward_batch_extend(ids[0, 7:], torch.tensor(slots), torch.tensor([12]), torch.tensor([5]),
                                          torch.tensor([7]), loc)
    got = mr2.forward(fb).next_token_logits
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)


def test_stacked_loader_and_tied_head():
    cfg = get_preset("qwen3-tiny")
    Model = get_model_class("Qwen3ForCausalLM")
    m = Model(cfg, params_dtype=torch.float32)
    H, D = cfg.hidden_size, cfg.head_dim
    sd = {
        "model.layers.0.self_attn.q_proj.weight": torch.full((4 * D, H), 1.0),
        "model.layers.0.self_attn.k_proj.weight": torch.full((2 * D, H), 2.0),
        "model.layers.0.self_attn.v_proj.weight": torch.full((2 * D, H), 3.0),
        "model.language_model.layers.1.mlp.gate_proj.weight": torch.full((512, H), 4.0),
        "model.language_model.layers.1.mlp.up_proj.weight": torch.full((512, H), 5.0),
        "lm_head.weight": torch.zeros(1024, H),  # ignored: embeddings are tied
    }
    loaded = m.load_weights(sd.items())
    w = m.model.layers[0].self_attn.qkv_proj.weight
    assert w[: 4 * D].eq(1).all() and w[4 * D: 6 * D].eq(2).all() and w[6 * D:].eq(3).all()
    gu = m.model.layers[1].mlp.gate_up_proj.weight
    assert gu[:512].eq(4).all() and gu[512:].eq(5).all()
    assert "lm_head.weight" not in loaded and m.lm_head_weight is m.model.embed_tokens.weight


def test_residual_carry_order():
    """The add of a block's output is folded into the next norm call, once per norm."""
    mr = _runner()
    calls = []
    from mllm_b200.layers import norm as norm_mod
    orig = norm_mod.RMSNorm.forward

    def spy(self, x, residual=None, **kw):
        calls.append(residual is not None)
        return orig(self, x, residual, **kw)

    norm_mod.RMSNorm.forward = spy
    try:
        _prefill(mr, torch.randint(0, 1024, (1, 4)))
    finally:
        norm_mod.RMSNorm.forward = orig
    # layer0.input (no residual yet), then every other norm incl. the final one carries the residual
    assert calls == [False] + [True] * (2 * 2 - 1) + [True]

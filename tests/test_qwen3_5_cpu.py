"""Qwen3.5 hybrid (gated delta net + gated attention) on CPU against HF transformers on a tiny config:
prefill, a chunked continuation of the prefill, and decode steps (which exercise the recurrent and
convolution state carried per request)."""
import types

import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner
from mllm_b200.ops import reference as ref


def test_gated_delta_rule_state_carry():
    torch.manual_seed(0)
    T, H, D = 7, 2, 8
    q, k, v = torch.randn(T, H, D), torch.randn(T, H, D), torch.randn(T, H, D)
    g, beta = -torch.rand(T, H), torch.rand(T, H)
    st = torch.zeros(3, H, D, D)
    idx = torch.tensor([1])
    whole = ref.gated_delta_rule(q, k, v, g, beta, st, idx, [T], [False])
    st2 = torch.zeros(3, H, D, D)
    a = ref.gated_delta_rule(q[:4], k[:4], v[:4], g[:4], beta[:4], st2, idx, [4], [False])
    b = ref.gated_delta_rule(q[4:], k[4:], v[4:], g[4:], beta[4:], st2, idx, [3], [True])
    torch.testing.assert_close(torch.cat([a, b]), whole)
    torch.testing.assert_close(st2[1], st[1])


def test_causal_conv_state_carry():
    torch.manual_seed(1)
    T, C, K = 9, 6, 4
    x, w = torch.randn(T, C), torch.randn(C, K)
    st = torch.zeros(2, C, K - 1)
    whole = ref.causal_conv1d_silu(x, w, st, torch.tensor([0]), [T], [False])
    st2 = torch.zeros(2, C, K - 1)
    a = ref.causal_conv1d_silu(x[:5], w, st2, torch.tensor([0]), [5], [False])
    b = ref.causal_conv1d_silu(x[5:], w, st2, torch.tensor([0]), [4], [True])
    torch.testing.assert_close(torch.cat([a, b]), whole)
    want = torch.nn.functional.silu(torch.nn.functional.conv1d(
        torch.nn.functional.pad(x.t().unsqueeze(0), (K - 1, 0)), w.unsqueeze(1), groups=C)).squeeze(0).t()
    torch.testing.assert_close(whole, want)


def test_matches_hf_qwen3_5():
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=2,
                num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256,
                attention_bias=False, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16,
                linear_num_key_heads=2, linear_num_value_heads=4, hidden_act="silu",
                layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                rope_parameters=dict(rope_theta=10000.0, partial_rotary_factor=0.25, rope_type="default", mrope_section=[2, 1, 1]))
    try:
        hf = tr.Qwen3_5ForCausalLM(tr.Qwen3_5TextConfig(**cfgd)).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3.5 unavailable: {e}")
    with torch.no_grad():   # make the zero-centred norm gains and decay parameters non-trivial
        for n, p in hf.named_parameters():
            if n.endswith(("layernorm.weight", "q_norm.weight", "k_norm.weight", "model.norm.weight")):
                p.copy_(torch.randn_like(p) * 0.1)
            if n.endswith("linear_attn.norm.weight"):
                p.copy_(1 + torch.randn_like(p) * 0.1)
    ns = types.SimpleNamespace(architectures=["Qwen3_5ForCausalLM"], **cfgd)
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    loaded = mr.model.load_weights(hf.state_dict().items())
    assert len(loaded) == len(dict(mr.model.named_parameters())), set(dict(mr.model.named_parameters())) - loaded
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    mr.model.post_load()
    torch.manual_seed(0)
    ids = torch.randint(0, 320, (1, 12))
    slots = mr.req_to_token_pool.alloc(1)
    sl = torch.tensor(slots)
    # prefill in two chunks (7 + 5 tokens): the second resumes from the stored conv / recurrent state
    loc = mr.token_to_kv_pool_allocator.alloc(12)
    mr.req_to_token_pool.req_to_token[slots[0], :12] = loc.int()
    fb = mr.prepare_forward_batch_extend(ids[0, :7], sl, torch.tensor([7]), torch.tensor([7]), torch.tensor([0]), loc[:7])
    mr.forward(fb)
    fb = mr.prepare_forward_batch_extend(ids[0, 7:], sl, torch.tensor([12]), torch.tensor([5]), torch.tensor([7]), loc[7:])
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)
    cur, seq = 12, ids
    for _ in range(2):
        nxt = got.argmax(-1)
        loc1 = mr.token_to_kv_pool_allocator.alloc(1)
        mr.req_to_token_pool.req_to_token[slots[0], cur] = loc1.int()
        cur += 1
        fbd = mr.prepare_forward_batch_decode(nxt, sl, torch.tensor([cur]), loc1)
        got = mr.forward(fbd).next_token_logits
        seq = torch.cat([seq, nxt[:, None]], 1)
        with torch.no_grad():
            want = hf(seq).logits[:, -1]
        torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)


def test_chunked_delta_rule_matches_the_token_loop():
    """The chunk-parallel (matrix product) form against the one-token-at-a-time definition: ragged
    batch, incoming state on some requests, several chunk sizes including one that leaves a short tail."""
    import torch

    from mllm_b200.ops import reference as ref

    torch.manual_seed(0)
    H, Dk, Dv = 4, 32, 48
    lens = [150, 7, 64, 129]
    T = sum(lens)
    q, k, v = torch.randn(T, H, Dk), torch.randn(T, H, Dk), torch.randn(T, H, Dv)
    g, beta = -torch.rand(T, H) * 0.3, torch.rand(T, H)
    st = torch.randn(6, H, Dk, Dv) * 0.1
    idx, has = torch.tensor([3, 0, 5, 1]), [1, 0, 1, 0]
    s_ref = st.clone()
    o_ref = ref.gated_delta_rule(q, k, v, g, beta, s_ref, idx, lens, has)
    for chunk in (16, 64, 128):
        s = st.clone()
        o = ref.gated_delta_rule_chunked(q, k, v, g, beta, s, idx, lens, has, chunk=chunk)
        assert (o - o_ref).abs().max() < 2e-6 and (s - s_ref).abs().max() < 2e-6
        assert torch.equal(s[2], st[2]) and torch.equal(s[4], st[4])   # rows of no request are untouched


def test_multimodal_variant_matches_hf():
    """Qwen3_5ForConditionalGeneration (vision tower + hybrid text model) against HF transformers on an
    image prompt: prefill logits, the image's position delta, and one decode step."""
    import types

    import pytest
    import torch

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner

    tr = pytest.importorskip("transformers")
    IMG, VSTART, VEND = 301, 302, 303
    text = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=2,
                num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256,
                attention_bias=False, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16,
                linear_num_key_heads=2, linear_num_value_heads=4, hidden_act="silu",
                layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                rope_parameters=dict(rope_theta=10000.0, partial_rotary_factor=0.5, rope_type="default", mrope_section=[4, 2, 2]))
    vision = dict(depth=2, hidden_size=32, hidden_act="gelu_pytorch_tanh", intermediate_size=64, num_heads=2, in_channels=3,
                  patch_size=16, spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=16)
    try:
        hf_cfg = tr.Qwen3_5Config(text_config=dict(text), vision_config=dict(vision), image_token_id=IMG, video_token_id=304,
                                  vision_start_token_id=VSTART, vision_end_token_id=VEND, tie_word_embeddings=False)
        hf = tr.Qwen3_5ForConditionalGeneration(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3.5 (multimodal) unavailable: {e}")
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(("layernorm.weight", "q_norm.weight", "k_norm.weight", "language_model.norm.weight")):
                p.copy_(torch.randn_like(p) * 0.1)
    ns = types.SimpleNamespace(architectures=["Qwen3_5ForConditionalGeneration"], model_type="qwen3_5", tie_word_embeddings=False,
                               image_token_id=IMG, video_token_id=304, vision_start_token_id=VSTART, vision_end_token_id=VEND,
                               text_config=types.SimpleNamespace(**text), vision_config=types.SimpleNamespace(**vision))
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    loaded = mr.model.load_weights(hf.state_dict().items())
    assert any(k.startswith("visual.") for k in loaded)
    missing = set(dict(mr.model.named_parameters())) - loaded
    assert not missing, missing
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    mr.model.post_load()
    torch.manual_seed(0)
    grid = torch.tensor([[1, 4, 6]])                     # 24 patches -> 6 merged tokens
    pixels = torch.randn(24, 3 * 2 * 16 * 16)
    ids = torch.tensor([[11, 12, VSTART] + [IMG] * 6 + [VEND, 13, 14, 15]])
    L = ids.shape[1]
    slots = mr.req_to_token_pool.alloc(1)
    loc = mr.token_to_kv_pool_allocator.alloc(L)
    mr.req_to_token_pool.req_to_token[slots[0], :L] = loc.int()
    lens = torch.tensor([L])
    fb = mr.prepare_forward_batch_extend(ids.reshape(-1), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc,
                                         pixel_values=pixels, image_grid_thw=grid)
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=(ids == IMG).int()).logits[:, -1]
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)
    assert fb.vit_prefill_tokens == 6 and int(fb.mrope_position_deltas[0]) == (3 + 3 + 4) - L
    nxt = got.argmax(-1)
    loc1 = mr.token_to_kv_pool_allocator.alloc(1)
    mr.req_to_token_pool.req_to_token[slots[0], L] = loc1.int()
    fbd = mr.prepare_forward_batch_decode(nxt, torch.tensor(slots), torch.tensor([L + 1]), loc1,
                                          mrope_position_deltas=fb.mrope_position_deltas)
    got2 = mr.forward(fbd).next_token_logits
    with torch.no_grad():
        ids2 = torch.cat([ids, nxt[:, None]], 1)
        want2 = hf(input_ids=ids2, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=(ids2 == IMG).int()).logits[:, -1]
    torch.testing.assert_close(got2, want2, atol=5e-4, rtol=5e-4)


def test_moe_variant_matches_hf():
    """Qwen3_5MoeForCausalLM: hybrid decoder with routed experts + gated shared expert in every layer,
    prefill in two chunks then decode, against HF transformers."""
    import types

    import pytest
    import torch

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner

    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1, head_dim=32,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256, attention_bias=False,
                linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                linear_num_value_heads=4, hidden_act="silu", moe_intermediate_size=32, shared_expert_intermediate_size=48,
                num_experts=4, num_experts_per_tok=2,
                layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                rope_parameters=dict(rope_theta=10000.0, partial_rotary_factor=0.25, rope_type="default", mrope_section=[2, 1, 1]))
    try:
        hf = tr.Qwen3_5MoeForCausalLM(tr.Qwen3_5MoeTextConfig(**cfgd)).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3.5-MoE unavailable: {e}")
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(("layernorm.weight", "q_norm.weight", "k_norm.weight", "model.norm.weight")):
                p.copy_(torch.randn_like(p) * 0.1)
            if n.endswith("mlp.gate.weight") or n.endswith("shared_expert_gate.weight"):
                p.copy_(torch.randn_like(p))
            if "experts" in n:
                p.copy_(torch.randn_like(p) * 0.05)
    ns = types.SimpleNamespace(architectures=["Qwen3_5MoeForCausalLM"], norm_topk_prob=True, **cfgd)
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    assert type(mr.model).__name__ == "Qwen3_5MoeForCausalLM"
    loaded = mr.model.load_weights(hf.state_dict().items())
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
    ids = torch.randint(0, 320, (1, 12))
    slots = mr.req_to_token_pool.alloc(1)
    sl = torch.tensor(slots)
    loc = mr.token_to_kv_pool_allocator.alloc(12)
    mr.req_to_token_pool.req_to_token[slots[0], :12] = loc.int()
    fb = mr.prepare_forward_batch_extend(ids[0, :7], sl, torch.tensor([7]), torch.tensor([7]), torch.tensor([0]), loc[:7])
    mr.forward(fb)
    fb = mr.prepare_forward_batch_extend(ids[0, 7:], sl, torch.tensor([12]), torch.tensor([5]), torch.tensor([7]), loc[7:])
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(got, want, atol=1e-3, rtol=1e-3)
    nxt = got.argmax(-1)
    loc1 = mr.token_to_kv_pool_allocator.alloc(1)
    mr.req_to_token_pool.req_to_token[slots[0], 12] = loc1.int()
    got = mr.forward(mr.prepare_forward_batch_decode(nxt, sl, torch.tensor([13]), loc1)).next_token_logits
    with torch.no_grad():
        want = hf(torch.cat([ids, nxt[:, None]], 1)).logits[:, -1]
    torch.testing.assert_close(got, want, atol=1e-3, rtol=1e-3)


def test_qwen3_next_matches_hf():
    """Qwen3-Next: fused per-key-head delta-net projections regrouped by the loader, one dense-MLP layer
    among the expert layers, 1-D rope."""
    import types

    import pytest
    import torch

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner

    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=2,
                num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256,
                attention_bias=False, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16,
                linear_num_key_heads=2, linear_num_value_heads=4, hidden_act="silu", moe_intermediate_size=32,
                shared_expert_intermediate_size=48, num_experts=4, num_experts_per_tok=2, norm_topk_prob=True,
                decoder_sparse_step=1, mlp_only_layers=[1],
                layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                rope_parameters=dict(rope_theta=10000.0, partial_rotary_factor=0.25, rope_type="default"))
    try:
        hf = tr.Qwen3NextForCausalLM(tr.Qwen3NextConfig(**cfgd)).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3-Next unavailable: {e}")
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(("layernorm.weight", "q_norm.weight", "k_norm.weight", "model.norm.weight")):
                p.copy_(torch.randn_like(p) * 0.1)
            if n.endswith("mlp.gate.weight") or n.endswith("shared_expert_gate.weight"):
                p.copy_(torch.randn_like(p))
            if "experts" in n:
                p.copy_(torch.randn_like(p) * 0.05)
    ns = types.SimpleNamespace(architectures=["Qwen3NextForCausalLM"], **cfgd)
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    assert type(mr.model.model.layers[1].mlp).__name__ == "MLP" and type(mr.model.model.layers[0].mlp).__name__ == "SharedExpertMoE"
    loaded = mr.model.load_weights(hf.state_dict().items())
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
    ids = torch.randint(0, 320, (1, 12))
    slots = mr.req_to_token_pool.alloc(1)
    sl = torch.tensor(slots)
    loc = mr.token_to_kv_pool_allocator.alloc(12)
    mr.req_to_token_pool.req_to_token[slots[0], :12] = loc.int()
    lens = torch.tensor([12])
    got = mr.forward(mr.prepare_forward_batch_extend(ids[0], sl, lens, lens, torch.zeros_like(lens), loc)).next_token_logits
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(got, want, atol=1e-3, rtol=1e-3)
    nxt = got.argmax(-1)
    loc1 = mr.token_to_kv_pool_allocator.alloc(1)
    mr.req_to_token_pool.req_to_token[slots[0], 12] = loc1.int()
    got = mr.forward(mr.prepare_forward_batch_decode(nxt, sl, torch.tensor([13]), loc1)).next_token_logits
    with torch.no_grad():
        want = hf(torch.cat([ids, nxt[:, None]], 1)).logits[:, -1]
    torch.testing.assert_close(got, want, atol=1e-3, rtol=1e-3)

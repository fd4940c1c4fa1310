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
                                     dict(rope_type="linear", factor=2.0),
                                     dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=16),
                                     dict(rope_type="yarn", factor=8.0, original_max_position_embeddings=32,
                                          beta_fast=16, beta_slow=2, mscale=1.0, mscale_all_dim=0.5),
                                     dict(rope_type="longrope", original_max_position_embeddings=16,
                                          short_factor=[1.0, 1.0, 1.1, 1.2, 1.3, 1.5, 1.8, 2.0],
                                          long_factor=[1.0, 1.2, 1.7, 2.5, 4.0, 7.0, 11.0, 16.0])])
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
                                num_key_value_heads=2, rms_norm_eps=1e-6, tie_word_embeddings=True, mlp_bias=True)
    with pytest.raises(NotImplementedError):
        get_model_class("LlamaForCausalLM")(cfg)
    cfg2 = types.SimpleNamespace(**{**vars(cfg), "mlp_bias": False, "rope_scaling": dict(rope_type="proportional", factor=4.0)})
    with pytest.raises(NotImplementedError):
        get_model_class("LlamaForCausalLM")(cfg2)


def test_mistral_sliding_window_matches_hf():
    """A window (8) much shorter than the prompt (40 tokens, prefilled in two chunks) and the decode steps."""
    tr = pytest.importorskip("transformers")
    cfgd = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
                hidden_act="silu", rope_theta=10000.0, sliding_window=8)
    try:
        hf = tr.MistralForCausalLM(tr.MistralConfig(**cfgd, attn_implementation="eager")).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Mistral unavailable: {e}")
    ns = types.SimpleNamespace(architectures=["MistralForCausalLM"], head_dim=16, **cfgd)
    _run_and_compare(hf, ns, 320)
    # the window matters: the same weights without it give other logits
    ns2 = types.SimpleNamespace(architectures=["MistralForCausalLM"], head_dim=16, **{**cfgd, "sliding_window": None})
    with pytest.raises(AssertionError):
        _run_and_compare(hf, ns2, 320)


def test_qwen2_window_layers_follow_max_window_layers():
    from mllm_b200.models.qwen3 import _sliding_window

    c = types.SimpleNamespace(sliding_window=16, use_sliding_window=True, max_window_layers=2)
    assert [_sliding_window(c, i) for i in range(4)] == [None, None, 16, 16]
    c.use_sliding_window = False
    assert _sliding_window(c, 3) is None
    c2 = types.SimpleNamespace(sliding_window=16, layer_types=["full_attention", "sliding_attention"])
    assert [_sliding_window(c2, i) for i in range(2)] == [None, 16]
    assert _sliding_window(types.SimpleNamespace(sliding_window=None), 0) is None


def test_qwen2_vl_matches_hf():
    """Qwen2-VL on an image prompt: translated vision tower (no position table, QuickGELU), sectioned 3-D rope."""
    tr = pytest.importorskip("transformers")
    IMG, VSTART, VEND = 301, 302, 303
    text = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-6, max_position_embeddings=256, hidden_act="silu", rope_theta=10000.0,
                rope_scaling=dict(type="mrope", mrope_section=[2, 3, 3]), tie_word_embeddings=False)
    vision = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, patch_size=14, spatial_merge_size=2,
                  temporal_patch_size=2, in_channels=3, hidden_act="quick_gelu")
    try:
        hf_cfg = tr.Qwen2VLConfig(text_config=dict(text), vision_config=dict(vision), image_token_id=IMG, video_token_id=304,
                                  vision_start_token_id=VSTART, vision_end_token_id=VEND, tie_word_embeddings=False)
        hf = tr.Qwen2VLForConditionalGeneration(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen2-VL unavailable: {e}")
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn_like(p) * 0.05)
    ns = types.SimpleNamespace(architectures=["Qwen2VLForConditionalGeneration"], model_type="qwen2_vl", tie_word_embeddings=False,
                               image_token_id=IMG, video_token_id=304, vision_start_token_id=VSTART, vision_end_token_id=VEND,
                               text_config=types.SimpleNamespace(head_dim=16, **text), vision_config=types.SimpleNamespace(**vision))
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    loaded = mr.model.load_weights(hf.state_dict().items())
    missing = {n for n in set(dict(mr.model.named_parameters())) - loaded if not n.endswith("patch_embed.proj.bias")}
    assert not missing, missing
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    torch.manual_seed(0)
    grid = torch.tensor([[1, 4, 6]])
    pixels = torch.randn(24, 3 * 2 * 14 * 14)
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
        try:
            want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=(ids == IMG).int()).logits[:, -1]
        except TypeError:
            want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid).logits[:, -1]
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)
    nxt = got.argmax(-1)
    loc1 = mr.token_to_kv_pool_allocator.alloc(1)
    mr.req_to_token_pool.req_to_token[slots[0], L] = loc1.int()
    fbd = mr.prepare_forward_batch_decode(nxt, torch.tensor(slots), torch.tensor([L + 1]), loc1,
                                          mrope_position_deltas=fb.mrope_position_deltas)
    got2 = mr.forward(fbd).next_token_logits
    with torch.no_grad():
        ids2 = torch.cat([ids, nxt[:, None]], 1)
        try:
            want2 = hf(input_ids=ids2, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=(ids2 == IMG).int()).logits[:, -1]
        except TypeError:
            want2 = hf(input_ids=ids2, pixel_values=pixels, image_grid_thw=grid).logits[:, -1]
    torch.testing.assert_close(got2, want2, atol=5e-4, rtol=5e-4)


def test_qwen2_5_vl_matches_hf():
    """Qwen2.5-VL: windowed vision attention (an image larger than one window, with ragged edge windows),
    one full-attention block, RMSNorm + SwiGLU tower, window order undone after the merger."""
    tr = pytest.importorskip("transformers")
    IMG, VSTART, VEND = 301, 302, 303
    text = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-6, max_position_embeddings=256, hidden_act="silu", rope_theta=10000.0,
                rope_scaling=dict(type="mrope", mrope_section=[2, 3, 3]), tie_word_embeddings=False)
    vision = dict(depth=3, hidden_size=32, hidden_act="silu", intermediate_size=48, num_heads=2, in_channels=3, patch_size=14,
                  spatial_merge_size=2, temporal_patch_size=2, window_size=56, out_hidden_size=64, fullatt_block_indexes=[1],
                  # An image is one temporal step, so its temporal position is the position where the image starts,
                  # as in the model's original definition.  The transformers version at hand multiplies that start
                  # position by tokens_per_second for images; 1 makes the two definitions coincide.
                  tokens_per_second=1)
    try:
        hf_cfg = tr.Qwen2_5_VLConfig(text_config=dict(text), vision_config=dict(vision), image_token_id=IMG, video_token_id=304,
                                     vision_start_token_id=VSTART, vision_end_token_id=VEND, tie_word_embeddings=False)
        hf = tr.Qwen2_5_VLForConditionalGeneration(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen2.5-VL unavailable: {e}")
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn_like(p) * 0.05)
            if "visual" in n and n.endswith(("norm1.weight", "norm2.weight", "ln_q.weight")):
                p.copy_(1 + torch.randn_like(p) * 0.1)
    ns = types.SimpleNamespace(architectures=["Qwen2_5_VLForConditionalGeneration"], model_type="qwen2_5_vl",
                               tie_word_embeddings=False, image_token_id=IMG, video_token_id=304, vision_start_token_id=VSTART,
                               vision_end_token_id=VEND, text_config=types.SimpleNamespace(head_dim=16, **text),
                               vision_config=types.SimpleNamespace(**vision))
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    loaded = mr.model.load_weights(hf.state_dict().items())
    missing = {n for n in set(dict(mr.model.named_parameters())) - loaded if not n.endswith("patch_embed.proj.bias")}
    assert not missing, missing
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    torch.manual_seed(0)
    grid = torch.tensor([[1, 6, 10]])                    # 3 x 5 merged tokens, windows of 2 x 2 merged tokens
    n_img = 15
    pixels = torch.randn(60, 3 * 2 * 14 * 14)
    ids = torch.tensor([[11, 12, VSTART] + [IMG] * n_img + [VEND, 13, 14, 15]])
    L = ids.shape[1]
    slots = mr.req_to_token_pool.alloc(1)
    loc = mr.token_to_kv_pool_allocator.alloc(L)
    mr.req_to_token_pool.req_to_token[slots[0], :L] = loc.int()
    lens = torch.tensor([L])
    fb = mr.prepare_forward_batch_extend(ids.reshape(-1), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc,
                                         pixel_values=pixels, image_grid_thw=grid)
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        feats = hf.model.visual(pixels, grid_thw=grid).pooler_output
        try:
            want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=(ids == IMG).int()).logits[:, -1]
        except TypeError:
            want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid).logits[:, -1]
    torch.testing.assert_close(mr.model.visual(pixels, grid), feats, atol=5e-4, rtol=5e-4)
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)

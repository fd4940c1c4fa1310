"""Qwen3-VL on CPU (fp32 PyTorch statements of the ops): position-id and interpolation helpers against
hand-computed values, and the whole model against HF transformers on a tiny random config."""
import types

import numpy as np
import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner
from mllm_b200.models.qwen3_vl import get_rope_index, interpolation_indices_and_weights, rot_pos_ids

IMG, VSTART = 1001, 1003


def test_get_rope_index_text_only():
    pos, delta = get_rope_index(torch.arange(5), None, IMG, VSTART, 2)
    assert pos.tolist() == [[0, 1, 2, 3, 4]] * 3 and delta == 0


def test_get_rope_index_with_image():
    # 2 text, <vision_start>, 1x4x4 grid -> 2x2 merged = 4 image tokens, 2 text
    ids = torch.tensor([5, 6, VSTART, IMG, IMG, IMG, IMG, 7, 8])
    pos, delta = get_rope_index(ids, [[1, 4, 4]], IMG, VSTART, 2)
    assert pos[0].tolist() == [0, 1, 2, 3, 3, 3, 3, 5, 6]
    assert pos[1].tolist() == [0, 1, 2, 3, 3, 4, 4, 5, 6]
    assert pos[2].tolist() == [0, 1, 2, 3, 4, 3, 4, 5, 6]
    assert delta == 7 - 9
    # continuing after a cached text prefix shifts everything
    pos2, delta2 = get_rope_index(ids, [[1, 4, 4]], IMG, VSTART, 2, start=10)
    assert (pos2 - pos == 10).all() and delta2 == delta


def test_rot_pos_ids_merge_order():
    ids = rot_pos_ids(4, 4, 2)
    # first merge group = the 2x2 block at the top-left corner
    assert ids[:4].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]]
    assert ids[4:8].tolist() == [[0, 2], [0, 3], [1, 2], [1, 3]]


def test_interpolation_weights_sum_to_one_and_hit_corners():
    idx, w = interpolation_indices_and_weights(3, 5, 8)
    assert np.allclose(sum(w), 1.0)
    assert idx[0][0] == 0 and np.isclose(w[0][0], 1.0)           # top-left sample sits on table entry 0
    assert idx[0][-1] == 63 or np.isclose(w[3][-1] + w[0][-1] + w[1][-1] + w[2][-1], 1.0)


def _tiny_cfg():
    text = dict(vocab_size=1100, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=2,
                num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6, rope_theta=5e6, max_position_embeddings=512,
                attention_bias=False, rope_scaling=dict(mrope_section=[24, 20, 20], mrope_interleaved=True, rope_type="default"))
    vision = dict(depth=3, hidden_size=64, num_heads=2, intermediate_size=96, patch_size=16, temporal_patch_size=2,
                  spatial_merge_size=2, in_channels=3, out_hidden_size=64, num_position_embeddings=64,
                  deepstack_visual_indexes=[0, 1], hidden_act="gelu_pytorch_tanh")
    return text, vision


def test_matches_hf_qwen3_vl():
    tr = pytest.importorskip("transformers")
    text, vision = _tiny_cfg()
    try:
        hf_cfg = tr.Qwen3VLConfig(text_config=dict(text), vision_config=dict(vision), image_token_id=IMG, video_token_id=1002,
                                  vision_start_token_id=VSTART, vision_end_token_id=1004, tie_word_embeddings=False)
        hf = tr.Qwen3VLForConditionalGeneration(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3-VL unavailable: {e}")
    ns = types.SimpleNamespace(architectures=["Qwen3VLForConditionalGeneration"], model_type="qwen3_vl",
                               tie_word_embeddings=False, image_token_id=IMG, video_token_id=1002,
                               vision_start_token_id=VSTART, vision_end_token_id=1004,
                               text_config=types.SimpleNamespace(tie_word_embeddings=False, **text),
                               vision_config=types.SimpleNamespace(**vision))
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=512),
                     hf_config=ns, device="cpu")
    mr.initialize()
    n_loaded = mr.model.load_weights(hf.state_dict().items())
    assert any(k.startswith("visual.") for k in n_loaded)
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    torch.manual_seed(0)
    grid = torch.tensor([[1, 4, 6]])                     # 24 patches -> 6 merged tokens
    pixels = torch.randn(24, 3 * 2 * 16 * 16)
    ids = torch.tensor([[11, 12, VSTART] + [IMG] * 6 + [1004, 13, 14, 15]])
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
    # one decode step with the stored delta
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


def test_matches_hf_qwen3_vl_moe():
    """Vision tower + deepstack + 3-D rope on the mixture-of-experts text model; the checkpoint keeps the
    experts of a layer fused in two 3-D tensors, which the loader splits."""
    tr = pytest.importorskip("transformers")
    text, vision = _tiny_cfg()
    text = dict(text, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2, norm_topk_prob=True,
                decoder_sparse_step=1, mlp_only_layers=[])
    try:
        hf_cfg = tr.Qwen3VLMoeConfig(text_config=dict(text), vision_config=dict(vision), image_token_id=IMG, video_token_id=1002,
                                     vision_start_token_id=VSTART, vision_end_token_id=1004, tie_word_embeddings=False)
        hf = tr.Qwen3VLMoeForConditionalGeneration(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3-VL-MoE unavailable: {e}")
    with torch.no_grad():   # spread the router so that different tokens pick different experts
        for n, p in hf.named_parameters():
            if n.endswith("mlp.gate.weight"):
                p.copy_(torch.randn_like(p))
            if "experts" in n:
                p.copy_(torch.randn_like(p) * 0.05)
    ns = types.SimpleNamespace(architectures=["Qwen3VLMoeForConditionalGeneration"], model_type="qwen3_vl_moe",
                               tie_word_embeddings=False, image_token_id=IMG, video_token_id=1002,
                               vision_start_token_id=VSTART, vision_end_token_id=1004,
                               text_config=types.SimpleNamespace(tie_word_embeddings=False, **text),
                               vision_config=types.SimpleNamespace(**vision))
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=512),
                     hf_config=ns, device="cpu")
    mr.initialize()
    assert type(mr.model).__name__ == "Qwen3VLMoeForConditionalGeneration"
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
    grid = torch.tensor([[1, 4, 6]])
    pixels = torch.randn(24, 3 * 2 * 16 * 16)
    ids = torch.tensor([[11, 12, VSTART] + [IMG] * 6 + [1004, 13, 14, 15]])
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
    torch.testing.assert_close(got, want, atol=1e-3, rtol=1e-3)


def test_builtin_image_preprocessing_matches_the_hf_processor():
    """Patch layout, grid and normalisation of the built-in image path against transformers' Qwen2-VL image
    processor: exact for a size that needs no resizing (both normalisation conventions); same grid and close
    pixels when a resize is involved (the resampling filters differ slightly)."""
    import numpy as np

    tr = pytest.importorskip("transformers")
    from mllm_b200.utils.image_processor import CLIP_MEAN, CLIP_STD, image_token_count, preprocess_image

    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, (320, 448, 3), dtype=np.uint8)
    for patch, mean, std in ((16, [0.5] * 3, [0.5] * 3), (14, list(CLIP_MEAN), list(CLIP_STD))):
        side = patch * 2
        im = img[: 10 * side, : 14 * side]
        hf = tr.Qwen2VLImageProcessor(patch_size=patch, merge_size=2, temporal_patch_size=2, image_mean=mean, image_std=std,
                                      min_pixels=64 * side * side, max_pixels=16384 * side * side)
        want = hf(images=[im], return_tensors="pt")
        pv, grid = preprocess_image(torch.from_numpy(im), patch, 2, 2, 64 * side * side, 16384 * side * side, mean, std)
        assert grid.tolist() == want["image_grid_thw"].tolist() and image_token_count(grid) == 10 * 14
        torch.testing.assert_close(pv, want["pixel_values"], atol=1e-5, rtol=1e-5)
    odd = rng.integers(0, 256, (211, 333, 3), dtype=np.uint8)
    hf = tr.Qwen2VLImageProcessor(patch_size=16, merge_size=2, temporal_patch_size=2, image_mean=[0.5] * 3, image_std=[0.5] * 3,
                                  min_pixels=64 * 32 * 32, max_pixels=16384 * 32 * 32)
    want = hf(images=[odd], return_tensors="pt")
    pv, grid = preprocess_image(torch.from_numpy(odd))
    assert grid.tolist() == want["image_grid_thw"].tolist() and pv.shape == want["pixel_values"].shape
    assert (pv - want["pixel_values"]).abs().mean().item() < 0.05

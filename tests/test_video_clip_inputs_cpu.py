"""Video inputs of the Qwen2-VL / Qwen2.5-VL families on CPU: one block per clip with grid ``[T, h, w]``, temporal
positions that advance per temporal patch (scaled by seconds x tokens_per_second for Qwen2.5-VL), frame sampling and
patch layout against transformers' video processor, the models against HF transformers on a clip, and requests
through the engine.

The 3-D positions follow the models' published definition: the temporal index of patch ``t`` is
``int(t * seconds_per_patch * tokens_per_second)`` (``t`` itself for Qwen2-VL), rows and columns count from the
block's first position, and text continues one past the largest position used.  The transformers version at hand
gives every temporal patch of a clip the same temporal index, so the HF models are run with these positions passed
in; everything else (tower over a ``[T, h, w]`` grid, feature placement, decoder) is HF's own."""
import types

import numpy as np
import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner
from mllm_b200.models.qwen3_vl import get_rope_index
from mllm_b200.orchestrator.tokenizer_process import TokenizerWorker
from mllm_b200.utils.image_processor import preprocess_video, sample_frame_indices_strided

IMG, VID, VSTART, VEND = 301, 304, 302, 303


def _published_positions(ids, grid, merge, step):
    """Positions of a prompt with one video block, written out from the definition."""
    t, h, w = grid[0], grid[1] // merge, grid[2] // merge
    pos, cur, i = [], 0, 0
    while i < len(ids):
        if ids[i] == VID:
            for a in range(t):
                for b in range(h):
                    for c in range(w):
                        pos.append((cur + int(a * step), cur + b, cur + c))
            cur = max(max(p) for p in pos[-t * h * w:]) + 1
            i += t * h * w
        else:
            pos.append((cur, cur, cur))
            cur += 1
            i += 1
    return torch.tensor(pos).T.contiguous(), cur - len(ids)


def test_rope_index_of_a_clip():
    ids = [11, VSTART] + [VID] * 12 + [VEND, 12]
    grid = [3, 4, 4]
    for step in (1.0, 50.0, 0.5, 2.5):
        want, delta = _published_positions(ids, grid, 2, step)
        got, d = get_rope_index(torch.tensor(ids), [grid], IMG, VSTART, 2, t_scales=[step])
        assert torch.equal(got, want) and d == delta, step
    # the example of the model's documentation: 3 temporal patches of 2 x 2 tokens, 50 positions per patch
    got, _ = get_rope_index(torch.tensor([VSTART] + [VID] * 12), [grid], IMG, VSTART, 2, t_scales=[50.0])
    assert (got[0, 1:] - 1).tolist() == [0] * 4 + [50] * 4 + [100] * 4
    assert (got[1, 1:] - 1).tolist() == [0, 0, 1, 1] * 3 and (got[2, 1:] - 1).tolist() == [0, 1, 0, 1] * 3
    # a cached text prefix shifts everything
    a, _ = get_rope_index(torch.tensor(ids), [grid], IMG, VSTART, 2, start=7, t_scales=[2.0])
    b, _ = get_rope_index(torch.tensor(ids), [grid], IMG, VSTART, 2, t_scales=[2.0])
    assert torch.equal(a, b + 7)


def test_strided_sampling_matches_the_hf_video_processor():
    tr = pytest.importorskip("transformers")
    try:
        from transformers.video_utils import VideoMetadata
        vp = tr.Qwen2VLVideoProcessor()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers video processor unavailable: {e}")
    for total, src in ((49, 24.0), (6, 3.0), (300, 30.0), (7, 24.0), (24 * 1000, 24.0)):
        want = vp.sample_frames(VideoMetadata(total_num_frames=total, fps=src), fps=2.0, min_frames=4, max_frames=768)
        got = sample_frame_indices_strided(total, src, 2.0, 4, 768, 2)
        assert got == [int(v) for v in want], (total, src)
    assert sample_frame_indices_strided(1, 24.0) == [0]


def test_clip_pixels_match_the_hf_video_processor():
    tr = pytest.importorskip("transformers")
    vid = np.random.default_rng(0).integers(0, 256, (5, 56, 84, 3), dtype=np.uint8)
    from mllm_b200.utils.image_processor import CLIP_MEAN, CLIP_STD
    try:
        vp = tr.Qwen2VLVideoProcessor(size={"shortest_edge": 28 * 28, "longest_edge": 768 * 28 * 28}, do_sample_frames=False)
        want = vp(videos=[torch.from_numpy(vid).permute(0, 3, 1, 2)], return_tensors="pt")
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers video processor unavailable: {e}")
    pv, grid = preprocess_video(torch.from_numpy(vid), 14, 2, 2, min_pixels=1, max_pixels=10 ** 9, mean=list(CLIP_MEAN),
                                std=list(CLIP_STD))
    assert grid.tolist() == want["video_grid_thw"].tolist() == [[3, 4, 6]]
    torch.testing.assert_close(pv, want["pixel_values_videos"], atol=1e-5, rtol=1e-5)


def test_builtin_clip_layout():
    mc = dict(image_token_id=IMG, video_token_id=VID, vision_start_token_id=VSTART, vision_end_token_id=VEND, patch_size=14,
              merge_size=2, temporal_patch_size=2, video_layout="clip", tokens_per_second=2.0)
    w = TokenizerWorker(None, vocab_size=300, mm_config=dict(mc))
    vid = np.random.default_rng(1).integers(0, 256, (12, 56, 84, 3), dtype=np.uint8)
    img = np.random.default_rng(2).integers(0, 256, (56, 56, 3), dtype=np.uint8)
    tok = w.tokenize({"rid": "r", "input_ids": [5, 6, 7], "video_data": {"frames": vid, "fps": 4.0}, "image_data": img})
    ids, mm = tok.input_ids, tok.mm_inputs
    grids = mm["image_grid_thw"].tolist()
    # 12 frames at 4 fps = 3 s -> 6 frames at 2 fps -> 3 temporal patches in ONE block; each spans 1 s = 2 positions
    assert len(grids) == 2 and grids[0][0] == 1 and grids[1][0] == 3
    per = (grids[1][1] // 2) * (grids[1][2] // 2)
    assert ids.count(VID) == 3 * per and ids.count(VSTART) == 2 and ids[-3:] == [5, 6, 7]
    first = ids.index(VID)
    assert ids[first - 1] == VSTART and ids[first:first + 3 * per] == [VID] * (3 * per) and ids[first + 3 * per] == VEND
    assert mm["mrope_t_scale"].tolist() == [1.0, 2.0]
    assert mm["pixel_values"].shape[0] == sum(g[0] * g[1] * g[2] for g in grids)
    # a placeholder in the text is replaced in place
    tok2 = w.tokenize({"rid": "r", "input_ids": [5, VSTART, VID, VEND, 6], "video_data": {"frames": vid, "fps": 4.0}})
    assert tok2.input_ids[0] == 5 and tok2.input_ids[-1] == 6 and tok2.input_ids.count(VID) == 3 * per
    # without tokens_per_second (Qwen2-VL) the positions advance by one per temporal patch
    w2 = TokenizerWorker(None, vocab_size=300, mm_config=dict(mc, tokens_per_second=None))
    assert "mrope_t_scale" not in w2.tokenize({"rid": "r", "input_ids": [5], "video_data": {"frames": vid, "fps": 4.0}}).mm_inputs
    # steps of a processor's videos are lined up with the merged grid list
    ipx, igr = torch.zeros(16, 1), torch.tensor([[1, 4, 4]])
    vpx, vgr = torch.zeros(48, 1), torch.tensor([[3, 4, 4]])
    pids = [VSTART] + [VID] * 12 + [VEND, VSTART] + [IMG] * 4 + [VEND]
    _, g, steps = TokenizerWorker.merge_vision_inputs(pids, ipx, igr, vpx, vgr, IMG, VID, VSTART, 2, video_steps=[4.0])
    assert g.tolist() == [[3, 4, 4], [1, 4, 4]] and steps.tolist() == [4.0, 1.0]


def _runner(ns):
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=256),
                     hf_config=ns, device="cpu")
    mr.initialize()
    return mr


def _finish_loading(mr, hf):
    loaded = mr.model.load_weights(hf.state_dict().items())
    missing = {n for n in set(dict(mr.model.named_parameters())) - loaded if not n.endswith("patch_embed.proj.bias")}
    assert not missing, missing
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)


def _clip_against_hf(mr, hf, grid, step, n_tok):
    torch.manual_seed(0)
    rows = grid[0] * grid[1] * grid[2]
    pixels = torch.randn(rows, 3 * 2 * 14 * 14)
    ids = torch.tensor([[11, 12, VSTART] + [VID] * n_tok + [VEND, 13, 14, 15]])
    L = ids.shape[1]
    slots = mr.req_to_token_pool.alloc(1)
    loc = mr.token_to_kv_pool_allocator.alloc(L)
    mr.req_to_token_pool.req_to_token[slots[0], :L] = loc.int()
    lens = torch.tensor([L])
    extra = {} if step == 1.0 else {"mrope_t_scale": torch.tensor([step], dtype=torch.float64)}
    fb = mr.prepare_forward_batch_extend(ids.reshape(-1), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc,
                                         pixel_values=pixels, image_grid_thw=torch.tensor([grid]), **extra)
    got = mr.forward(fb).next_token_logits
    pos, delta = _published_positions(ids[0].tolist(), grid, 2, step)
    assert torch.equal(fb.mrope_positions.cpu(), pos) and int(fb.mrope_position_deltas[0]) == delta
    vgrid = torch.tensor([grid])
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values_videos=pixels, video_grid_thw=vgrid, position_ids=pos[:, None, :],
                  mm_token_type_ids=(ids == VID).int() * 2).logits[:, -1]
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)
    assert fb.vit_prefill_tokens == n_tok
    # one decode step: the next position is the prompt's length plus the delta
    nxt = got.argmax(-1)
    loc1 = mr.token_to_kv_pool_allocator.alloc(1)
    mr.req_to_token_pool.req_to_token[slots[0], L] = loc1.int()
    fbd = mr.prepare_forward_batch_decode(nxt, torch.tensor(slots), torch.tensor([L + 1]), loc1,
                                          mrope_position_deltas=fb.mrope_position_deltas)
    got2 = mr.forward(fbd).next_token_logits
    ids2 = torch.cat([ids, nxt[:, None]], 1)
    pos2 = torch.cat([pos, torch.full((3, 1), L + delta)], 1)
    with torch.no_grad():
        want2 = hf(input_ids=ids2, pixel_values_videos=pixels, video_grid_thw=vgrid, position_ids=pos2[:, None, :],
                   mm_token_type_ids=(ids2 == VID).int() * 2).logits[:, -1]
    torch.testing.assert_close(got2, want2, atol=5e-4, rtol=5e-4)


_TEXT = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, rms_norm_eps=1e-6, max_position_embeddings=256, hidden_act="silu", rope_theta=10000.0,
             rope_scaling=dict(type="mrope", mrope_section=[2, 3, 3]), tie_word_embeddings=False)


def test_qwen2_vl_matches_hf_on_a_clip():
    tr = pytest.importorskip("transformers")
    vision = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, patch_size=14, spatial_merge_size=2,
                  temporal_patch_size=2, in_channels=3, hidden_act="quick_gelu")
    try:
        hf_cfg = tr.Qwen2VLConfig(text_config=dict(_TEXT), vision_config=dict(vision), image_token_id=IMG, video_token_id=VID,
                                  vision_start_token_id=VSTART, vision_end_token_id=VEND, tie_word_embeddings=False)
        hf = tr.Qwen2VLForConditionalGeneration(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen2-VL unavailable: {e}")
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn_like(p) * 0.05)
    ns = types.SimpleNamespace(architectures=["Qwen2VLForConditionalGeneration"], model_type="qwen2_vl", tie_word_embeddings=False,
                               image_token_id=IMG, video_token_id=VID, vision_start_token_id=VSTART, vision_end_token_id=VEND,
                               text_config=types.SimpleNamespace(head_dim=16, **_TEXT), vision_config=types.SimpleNamespace(**vision))
    mr = _runner(ns)
    _finish_loading(mr, hf)
    _clip_against_hf(mr, hf, [3, 4, 6], 1.0, 18)


def test_qwen2_5_vl_matches_hf_on_a_clip():
    """Three temporal patches, each larger than one attention window; the temporal position advances by 2 per patch."""
    tr = pytest.importorskip("transformers")
    vision = dict(depth=3, hidden_size=32, hidden_act="silu", intermediate_size=48, num_heads=2, in_channels=3, patch_size=14,
                  spatial_merge_size=2, temporal_patch_size=2, window_size=56, out_hidden_size=64, fullatt_block_indexes=[1],
                  tokens_per_second=2)
    try:
        hf_cfg = tr.Qwen2_5_VLConfig(text_config=dict(_TEXT), vision_config=dict(vision), image_token_id=IMG, video_token_id=VID,
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
                               tie_word_embeddings=False, image_token_id=IMG, video_token_id=VID, vision_start_token_id=VSTART,
                               vision_end_token_id=VEND, text_config=types.SimpleNamespace(head_dim=16, **_TEXT),
                               vision_config=types.SimpleNamespace(**vision))
    mr = _runner(ns)
    _finish_loading(mr, hf)
    _clip_against_hf(mr, hf, [3, 6, 10], 2.0, 45)


@pytest.mark.parametrize("preset", ["qwen2-vl-tiny", "qwen2.5-vl-tiny"])
def test_clip_request_through_the_engine(preset):
    from mllm_b200.engine.launch import Engine

    cfg = ServerConfig(model_path=f"preset:{preset}", dtype="float32", max_running_requests=2, max_total_tokens=4096,
                       context_length=2048, log_level="warning", chunked_prefill_size=64)
    eng = Engine(cfg, mode="inproc", device="cpu").launch()
    try:
        vid = np.random.default_rng(0).integers(0, 256, (6, 56, 84, 3), dtype=np.uint8)
        img = np.random.default_rng(1).integers(0, 256, (56, 56, 3), dtype=np.uint8)
        sp = {"max_new_tokens": 4, "temperature": 0.0}
        a = eng.generate("what happens", sp, video_data={"frames": vid, "fps": 3.0})
        b = eng.generate("what happens", sp, video_data={"frames": list(vid), "fps": 3.0})
        assert len(a["output_ids"]) == 4 and a["output_ids"] == b["output_ids"]
        c = eng.generate("what happens", sp, video_data={"frames": vid, "fps": 3.0}, image_data=img)
        assert c["meta_info"]["prompt_tokens"] > a["meta_info"]["prompt_tokens"] and len(c["output_ids"]) == 4
        tok = eng.tokenizer_worker.tokenize({"rid": "x", "text": "what happens", "video_data": {"frames": vid, "fps": 3.0}})
        assert tok.mm_inputs["image_grid_thw"][0, 0] == 2
        assert ("mrope_t_scale" in tok.mm_inputs) == (preset == "qwen2.5-vl-tiny")
    finally:
        eng.shutdown()


def test_temporal_steps_stay_aligned_with_the_grids_of_a_mixed_batch():
    """An image request (no step list) and a clip request (steps) prefilled in one pass: one step per grid, in order."""
    from mllm_b200.orchestrator.model_runner_process import ModelRunnerProcess

    me = types.SimpleNamespace(device=torch.device("cpu"))
    img = types.SimpleNamespace(mm_inputs={"pixel_values": torch.zeros(16, 4), "image_grid_thw": torch.tensor([[1, 4, 4]])})
    clip = types.SimpleNamespace(mm_inputs={"pixel_values": torch.zeros(48 + 16, 4),
                                            "image_grid_thw": torch.tensor([[3, 4, 4], [1, 4, 4]]),
                                            "mrope_t_scale": torch.tensor([2.0, 1.0], dtype=torch.float64)})
    text = types.SimpleNamespace(mm_inputs=None)
    out = ModelRunnerProcess._mm_kwargs(me, [(img, 0), (text, 0), (clip, 0)])
    assert out["image_grid_thw"].tolist() == [[1, 4, 4], [3, 4, 4], [1, 4, 4]] and out["pixel_values"].shape[0] == 80
    assert out["mrope_t_scale"].tolist() == [1.0, 2.0, 1.0]
    # consumed once: a second pass over the same requests carries no pixels
    assert ModelRunnerProcess._mm_kwargs(me, [(img, 0), (clip, 0)]) == {}
    only_images = types.SimpleNamespace(mm_inputs={"pixel_values": torch.zeros(16, 4), "image_grid_thw": torch.tensor([[1, 4, 4]])})
    assert "mrope_t_scale" not in ModelRunnerProcess._mm_kwargs(me, [(only_images, 0)])

"""Video inputs of the Qwen3-VL family on CPU: frame preprocessing against transformers' video processor,
timestamps, the prompt layout (one timestamped block per temporal patch), merging of a processor's separate
image / video outputs, the model against HF transformers on a clip, and a request through the engine."""
import types

import numpy as np
import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner
from mllm_b200.orchestrator.tokenizer_process import TokenizerWorker
from mllm_b200.utils.image_processor import preprocess_video, sample_frame_indices, video_timestamps

IMG, VID, VSTART, VEND = 1001, 1002, 1003, 1004
MC = dict(image_token_id=IMG, video_token_id=VID, vision_start_token_id=VSTART, vision_end_token_id=VEND, patch_size=16,
          merge_size=2, temporal_patch_size=2, video_min_frames=2)


def test_frames_match_the_hf_video_processor():
    tr = pytest.importorskip("transformers")
    vid = np.random.default_rng(0).integers(0, 256, (5, 64, 96, 3), dtype=np.uint8)      # odd count: last frame repeated
    try:
        vp = tr.Qwen3VLVideoProcessor(patch_size=16, merge_size=2, temporal_patch_size=2, image_mean=[0.5] * 3,
                                      image_std=[0.5] * 3, size={"shortest_edge": 1024, "longest_edge": 768 * 32 * 32},
                                      do_sample_frames=False)
        want = vp(videos=[torch.from_numpy(vid).permute(0, 3, 1, 2)], return_tensors="pt")
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers video processor unavailable: {e}")
    pv, grid = preprocess_video(torch.from_numpy(vid), min_pixels=1, max_pixels=10 ** 9)
    assert grid.tolist() == want["video_grid_thw"].tolist() == [[3, 4, 6]]
    torch.testing.assert_close(pv, want["pixel_values_videos"], atol=1e-5, rtol=1e-5)


def test_sampling_and_timestamps():
    assert sample_frame_indices(49, 24.0, 2.0, min_frames=4, max_frames=768) == [0, 16, 32, 48]     # 2 s clip at 2 fps
    assert sample_frame_indices(3, 24.0, 2.0, min_frames=4) == [0, 1, 2]                            # short clip: all frames
    assert len(sample_frame_indices(24 * 1000, 24.0, 2.0, max_frames=100)) == 100
    assert video_timestamps([0, 12, 24, 36, 48], 24.0, 2) == [0.25, 1.25, 2.0]


def _worker():
    w = TokenizerWorker(None, vocab_size=1000, mm_config=dict(MC))
    return w


def test_builtin_video_prompt_layout_and_placeholders():
    w = _worker()
    vid = np.random.default_rng(1).integers(0, 256, (4, 64, 96, 3), dtype=np.uint8)
    img = np.random.default_rng(2).integers(0, 256, (64, 64, 3), dtype=np.uint8)
    req = {"rid": "r", "input_ids": [5, 6, 7], "video_data": {"frames": vid, "fps": 2.0}, "image_data": img}
    tok = w.tokenize(req)
    ids, mm = tok.input_ids, tok.mm_inputs
    grids = mm["image_grid_thw"].tolist()
    assert grids[0][0] == 1 and len(grids) == 3 and grids[1] == grids[2] and grids[1][0] == 1    # image, then 2 temporal patches
    per = (grids[1][1] // 2) * (grids[1][2] // 2)
    assert ids.count(VID) == 2 * per and ids.count(VSTART) == 3 and ids[-3:] == [5, 6, 7]
    assert mm["pixel_values"].shape[0] == sum(g[0] * g[1] * g[2] for g in grids)
    # the timestamps "<0.2 seconds>" / "<1.2 seconds>" sit in front of each block
    stamp = w.tokenizer.encode("<0.2 seconds>")
    first_video_block = ids.index(VID) - 1
    assert ids[first_video_block - len(stamp):first_video_block] == stamp
    # placeholders written by a chat template are replaced in place, in order of appearance: video first here
    req2 = dict(req, input_ids=[5, VSTART, VID, VEND, 6, VSTART, IMG, VEND, 7])
    tok2 = w.tokenize(req2)
    ids2, g2 = tok2.input_ids, tok2.mm_inputs["image_grid_thw"].tolist()
    assert ids2[0] == 5 and ids2[-1] == 7 and ids2.count(VSTART) == 3
    assert ids2.index(VID) < ids2.index(IMG) and g2 == [grids[1], grids[2], grids[0]]
    assert tok2.mm_inputs["pixel_values"].shape == mm["pixel_values"].shape
    with pytest.raises(ValueError, match="mp4"):
        w.tokenize({"rid": "r", "text": "x", "video_data": "clip.mp4"})
    no_video = TokenizerWorker(None, vocab_size=1000, mm_config=dict(MC, video_token_id=None))
    with pytest.raises(ValueError, match="no video token"):
        no_video.tokenize({"rid": "r", "text": "x", "video_data": vid})


def test_merge_of_separate_image_and_video_outputs():
    ipx, igr = torch.arange(16.0).view(16, 1), torch.tensor([[1, 4, 4]])
    vpx, vgr = 100 + torch.arange(48.0).view(48, 1), torch.tensor([[3, 4, 4]])
    blk = lambda tok, n: [VSTART] + [tok] * n + [VEND]  # noqa: E731
    # one block per temporal patch (Qwen3-VL layout), the image between the second and the third
    ids = [1] + blk(VID, 4) + [2] + blk(VID, 4) + blk(IMG, 4) + [3] + blk(VID, 4)
    pv, g = TokenizerWorker.merge_vision_inputs(ids, ipx, igr, vpx, vgr, IMG, VID, VSTART, 2)
    assert g.tolist() == [[1, 4, 4], [1, 4, 4], [1, 4, 4], [1, 4, 4]]
    assert pv.flatten().tolist() == list(range(100, 132)) + list(range(16)) + list(range(132, 148))
    # the whole clip in one block
    ids = blk(IMG, 4) + blk(VID, 12)
    pv, g = TokenizerWorker.merge_vision_inputs(ids, ipx, igr, vpx, vgr, IMG, VID, VSTART, 2)
    assert g.tolist() == [[1, 4, 4], [3, 4, 4]] and pv.shape[0] == 64


def test_model_matches_hf_on_a_clip():
    tr = pytest.importorskip("transformers")
    text = dict(vocab_size=1100, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=2,
                num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6, rope_theta=5e6, max_position_embeddings=512,
                attention_bias=False, rope_scaling=dict(mrope_section=[24, 20, 20], mrope_interleaved=True, rope_type="default"))
    vision = dict(depth=3, hidden_size=64, num_heads=2, intermediate_size=96, patch_size=16, temporal_patch_size=2,
                  spatial_merge_size=2, in_channels=3, out_hidden_size=64, num_position_embeddings=64,
                  deepstack_visual_indexes=[0, 1], hidden_act="gelu_pytorch_tanh")
    try:
        hf_cfg = tr.Qwen3VLConfig(text_config=dict(text), vision_config=dict(vision), image_token_id=IMG, video_token_id=VID,
                                  vision_start_token_id=VSTART, vision_end_token_id=VEND, tie_word_embeddings=False)
        hf = tr.Qwen3VLForConditionalGeneration(hf_cfg).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers Qwen3-VL unavailable: {e}")
    ns = types.SimpleNamespace(architectures=["Qwen3VLForConditionalGeneration"], model_type="qwen3_vl",
                               tie_word_embeddings=False, image_token_id=IMG, video_token_id=VID,
                               vision_start_token_id=VSTART, vision_end_token_id=VEND,
                               text_config=types.SimpleNamespace(tie_word_embeddings=False, **text),
                               vision_config=types.SimpleNamespace(**vision))
    mr = ModelRunner(ServerConfig(model_path="preset:x", dtype="float32", max_running_requests=2, max_total_tokens=512),
                     hf_config=ns, device="cpu")
    mr.initialize()
    mr.model.load_weights(hf.state_dict().items())
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    torch.manual_seed(0)
    pixels = torch.randn(2 * 24, 3 * 2 * 16 * 16)                      # two temporal patches of 4 x 6 patches
    blk = [VSTART] + [VID] * 6 + [VEND]
    ids = torch.tensor([[11, 12, 20, 21] + blk + [22, 23] + blk + [13, 14, 15]])
    L = ids.shape[1]
    slots = mr.req_to_token_pool.alloc(1)
    loc = mr.token_to_kv_pool_allocator.alloc(L)
    mr.req_to_token_pool.req_to_token[slots[0], :L] = loc.int()
    lens = torch.tensor([L])
    fb = mr.prepare_forward_batch_extend(ids.reshape(-1), torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc,
                                         pixel_values=pixels, image_grid_thw=torch.tensor([[1, 4, 6], [1, 4, 6]]))
    got = mr.forward(fb).next_token_logits
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values_videos=pixels, video_grid_thw=torch.tensor([[2, 4, 6]]),
                  mm_token_type_ids=(ids == VID).int() * 2).logits[:, -1]
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)
    assert fb.vit_prefill_tokens == 12


def test_video_request_through_the_engine():
    from mllm_b200.engine.launch import Engine

    cfg = ServerConfig(model_path="preset:qwen3-vl-tiny", dtype="float32", max_running_requests=2, max_total_tokens=2048,
                       context_length=1024, log_level="warning", chunked_prefill_size=64)
    eng = Engine(cfg, mode="inproc", device="cpu").launch()
    try:
        vid = np.random.default_rng(0).integers(0, 256, (6, 64, 96, 3), dtype=np.uint8)
        sp = {"max_new_tokens": 4, "temperature": 0.0}
        a = eng.generate("what happens", sp, video_data={"frames": vid, "fps": 3.0})
        b = eng.generate("what happens", sp, video_data={"frames": list(vid), "fps": 3.0})       # frames as a list
        assert len(a["output_ids"]) == 4 and a["output_ids"] == b["output_ids"]
        c = eng.generate("what happens", sp, video_data={"frames": vid[::-1].copy(), "fps": 3.0})
        assert c["meta_info"]["prompt_tokens"] == a["meta_info"]["prompt_tokens"]
    finally:
        eng.shutdown()


def test_video_and_image_parts_over_http(tmp_path):
    testclient = pytest.importorskip("fastapi.testclient")
    from mllm_b200.configs import GlobalConfig
    from mllm_b200.engine.launch import Engine
    from mllm_b200.server.launch import create_app

    GlobalConfig.reset()
    cfg = ServerConfig(model_path="preset:qwen3-vl-tiny", dtype="float32", max_running_requests=2, max_total_tokens=4096,
                       context_length=2048, log_level="warning")
    eng = Engine(cfg, mode="inproc", device="cpu").launch()
    try:
        rng = np.random.default_rng(0)
        vid = rng.integers(0, 256, (4, 64, 64, 3), dtype=np.uint8)
        img = rng.integers(0, 256, (64, 64, 3), dtype=np.uint8)
        with testclient.TestClient(create_app(eng)) as c:
            msgs = [{"role": "user", "content": [
                {"type": "video", "video": {"frames": vid.tolist(), "fps": 2.0}},
                {"type": "image", "image": img.tolist()},
                {"type": "text", "text": "compare"}]}]
            r = c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 3, "temperature": 0})
            assert r.status_code == 200, r.text
            usage = r.json()["usage"]
            tok = eng.tokenizer_worker.tokenize({"rid": "x", "text": "compare", "video_data": {"frames": vid, "fps": 2.0},
                                                 "image_data": img})
            n_vision = sum(1 for t in tok.input_ids if t in (IMG, VID))
            assert usage["completion_tokens"] == 3 and usage["prompt_tokens"] > n_vision > 0
            clip = _write_clip(tmp_path / "clip.mp4")
            import base64
            uri = "data:video/mp4;base64," + base64.b64encode(clip.read_bytes()).decode()
            for url in (uri, "file://" + str(clip)):
                msgs = [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": url}}, {"type": "text", "text": "go"}]}]
                r = c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 2, "temperature": 0})
                assert r.status_code == 200, r.text
                assert r.json()["usage"]["prompt_tokens"] > 20
            r = c.post("/generate", json={"text": "what", "video_data": {"frames": vid.tolist(), "fps": 2.0},
                                          "sampling_params": {"max_new_tokens": 2, "temperature": 0}})
            assert r.status_code == 200 and r.json()["meta_info"]["completion_tokens"] == 2
    finally:
        eng.shutdown()


def _write_clip(path, n=12, fps=10.0, size=(96, 64), step=20):
    cv2 = pytest.importorskip("cv2")
    w = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"mp4v"), fps, size)
    if not w.isOpened():
        pytest.skip("this OpenCV build cannot write mp4")
    for i in range(n):
        w.write(np.full((size[1], size[0], 3), i * step, dtype=np.uint8))     # frame i is a flat grey of value step x i
    w.release()
    return path


def test_container_files_are_decoded_and_only_the_sampled_frames_are_converted(tmp_path):
    """An mp4 written here is read back through the OpenCV reader: all frames, or just the sampled frame numbers."""
    clip = _write_clip(tmp_path / "clip.mp4")
    frames, fps = TokenizerWorker.load_video(str(clip))
    assert tuple(frames.shape) == (12, 64, 96, 3) and fps == 10.0
    level = frames.float().mean(dim=(1, 2, 3))
    assert (level - torch.arange(12) * 20.0).abs().max() < 6                     # lossy codec: close, in order
    kept, keep, src_fps, total = TokenizerWorker.load_video_sampled(str(clip), lambda n, f: [0, 5, 5, 11])
    assert keep == [0, 5, 5, 11] and total == 12 and src_fps == 10.0 and kept.shape[0] == 4
    assert (kept.float().mean(dim=(1, 2, 3)) - torch.tensor([0.0, 100.0, 100.0, 220.0])).abs().max() < 6
    # the same file as bytes, as a data URI, and with a rate that overrides the container's
    raw = clip.read_bytes()
    import base64
    for item in (raw, "data:video/mp4;base64," + base64.b64encode(raw).decode(), {"frames": str(clip), "fps": 5.0}):
        f2, fps2 = TokenizerWorker.load_video(item)
        assert f2.shape == frames.shape and fps2 == (5.0 if isinstance(item, dict) else 10.0)
    with pytest.raises(ValueError, match="neither"):
        TokenizerWorker.load_video("clip.txt")
    with pytest.raises(ValueError, match="cannot open"):
        TokenizerWorker.load_video(str(tmp_path / "missing.mp4"))


def test_container_request_matches_the_same_frames_given_as_an_array(tmp_path):
    clip = _write_clip(tmp_path / "clip.mp4", n=20, fps=10.0, step=12)
    w = _worker()
    frames, fps = TokenizerWorker.load_video(str(clip))
    a = w.tokenize({"rid": "a", "input_ids": [5], "video_data": str(clip)})
    b = w.tokenize({"rid": "b", "input_ids": [5], "video_data": {"frames": frames.numpy(), "fps": fps}})
    assert a.input_ids == b.input_ids
    assert torch.equal(a.mm_inputs["pixel_values"], b.mm_inputs["pixel_values"])
    assert a.mm_inputs["image_grid_thw"].tolist() == b.mm_inputs["image_grid_thw"].tolist()
    two = w.tokenize({"rid": "c", "input_ids": [5], "video_data": [str(clip), str(clip)]})      # a list of containers = two videos
    assert two.mm_inputs["pixel_values"].shape[0] == 2 * a.mm_inputs["pixel_values"].shape[0]


def test_remote_image_and_clip_urls_are_fetched_with_limits(tmp_path, monkeypatch):
    """A local HTTP server stands in for the remote host."""
    import functools
    import http.server
    import threading

    from PIL import Image

    img = np.random.default_rng(3).integers(0, 256, (40, 48, 3), dtype=np.uint8)
    Image.fromarray(img).save(tmp_path / "pic.png")
    clip = _write_clip(tmp_path / "clip.mp4")
    handler = functools.partial(http.server.SimpleHTTPRequestHandler, directory=str(tmp_path))
    handler.log_message = lambda *a, **k: None
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), handler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{srv.server_address[1]}"
    monkeypatch.setenv("no_proxy", "127.0.0.1")          # a proxy configured for the machine must not see this
    monkeypatch.setenv("NO_PROXY", "127.0.0.1")
    try:
        got = np.asarray(TokenizerWorker.load_image(base + "/pic.png"))
        assert np.array_equal(got, img)
        assert np.array_equal(np.asarray(TokenizerWorker.load_image("file://" + str(tmp_path / "pic.png"))), img)
        frames, fps = TokenizerWorker.load_video(base + "/clip.mp4")
        assert tuple(frames.shape) == (12, 64, 96, 3) and fps == 10.0
        with pytest.raises(ValueError, match="could not fetch"):
            TokenizerWorker.load_image(base + "/missing.png")
        monkeypatch.setattr(TokenizerWorker, "_FETCH_MAX_BYTES", 100)
        with pytest.raises(ValueError, match="larger than"):
            TokenizerWorker.load_image(base + "/pic.png")
        monkeypatch.setenv("MLLM_B200_FETCH_URLS", "0")
        with pytest.raises(ValueError, match="disabled"):
            TokenizerWorker.load_image(base + "/pic.png")
    finally:
        srv.shutdown()

"""The Qwen2-VL / Qwen2.5-VL presets are valid inputs of the transformers config classes of their families, and a
transformers model built from a preset and the engine's model built from the same preset give the same logits on
an image prompt (the presets' field names and shapes are the checkpoints' own)."""
import copy

import pytest
import torch

from mllm_b200.configs import ServerConfig
from mllm_b200.executor import ModelRunner
from mllm_b200.models.presets import PRESETS, get_preset, preset_to_config_json


@pytest.mark.parametrize("name,cfg_cls,model_cls", [
    ("qwen2-vl-tiny", "Qwen2VLConfig", "Qwen2VLForConditionalGeneration"),
    ("qwen2.5-vl-tiny", "Qwen2_5_VLConfig", "Qwen2_5_VLForConditionalGeneration"),
])
def test_tiny_preset_against_transformers(name, cfg_cls, model_cls):
    tr = pytest.importorskip("transformers")
    d = preset_to_config_json(name)
    for k in ("architectures", "torch_dtype", "model_type"):
        d.pop(k, None)
    # An image is one temporal step: its temporal position is where the block starts.  The transformers version
    # at hand multiplies that start by tokens_per_second; 1 makes the two definitions coincide (clips are compared
    # with explicit positions elsewhere).
    overrides = {}
    if "tokens_per_second" in d["vision_config"]:
        d["vision_config"]["tokens_per_second"] = 1
        overrides["vision_config"] = dict(d["vision_config"])
    try:
        hf = getattr(tr, model_cls)(getattr(tr, cfg_cls)(**copy.deepcopy(d))).float().eval()
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers cannot build {model_cls}: {e}")
    mr = ModelRunner(ServerConfig(model_path=f"preset:{name}", dtype="float32", max_running_requests=2, max_total_tokens=512),
                     hf_config=get_preset(name, **overrides), device="cpu")
    mr.initialize()
    loaded = mr.model.load_weights(hf.state_dict().items())
    missing = {n for n in set(dict(mr.model.named_parameters())) - loaded if not n.endswith("patch_embed.proj.bias")}
    assert not missing, missing
    for m in mr.model.modules():
        if hasattr(m, "quant_method"):
            m._gate_up_interleaved = False
            m.quant_method.process_weights_after_loading(m)
    IMG, VS, VE = d["image_token_id"], d["vision_start_token_id"], d["vision_end_token_id"]
    torch.manual_seed(0)
    grid = torch.tensor([[1, 4, 6]])
    pixels = torch.randn(24, 3 * 2 * 14 * 14)
    ids = torch.tensor([[11, 12, VS] + [IMG] * 6 + [VE, 13, 14]])
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


@pytest.mark.parametrize("name,cfg_cls", [("qwen2-vl-2b", "Qwen2VLConfig"), ("qwen2.5-vl-3b", "Qwen2_5_VLConfig")])
def test_published_shapes_are_accepted_by_the_config_classes(name, cfg_cls):
    tr = pytest.importorskip("transformers")
    d = copy.deepcopy(PRESETS[name])
    for k in ("architectures", "torch_dtype", "model_type"):
        d.pop(k, None)
    cfg = getattr(tr, cfg_cls)(**d)
    tc = cfg.text_config if hasattr(cfg, "text_config") else cfg
    assert tc.hidden_size == d["text_config"]["hidden_size"] and tc.num_hidden_layers == d["text_config"]["num_hidden_layers"]
    assert cfg.vision_config.depth == d["vision_config"]["depth"] and cfg.image_token_id == d["image_token_id"]

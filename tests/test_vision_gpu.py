"""Vision-tower kernels and the Qwen3-VL model on the GPU against the fp32 PyTorch statements."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,H,lens", [(64, 16, [784]), (64, 4, [100, 36, 260]), (128, 2, [130, 7]), (72, 3, [64, 200])])
def test_vision_attention(D, H, lens):
    torch.manual_seed(D + H)
    T = sum(lens)
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(torch.bfloat16)
    ang = torch.rand(T, D // 2, device="cuda") * 6.28
    cos, sin = ang.cos(), ang.sin()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    got = ops.vision_attention(qkv, cos, sin, cu, H, D ** -0.5).float()
    q, k, v = qkv.view(T, 3, H, D).float().unbind(1)
    q, k = ref.vision_rope(q, cos, sin), ref.vision_rope(k, cos, sin)
    want = ref.attention_varlen_bidirectional(q, k, v, cu, D ** -0.5).reshape(T, H * D)
    ops.check_status()
    assert (got - want).abs().max().item() < 0.03


def test_varlen_bidirectional_plain():
    torch.manual_seed(1)
    T, H, D = 300, 4, 64
    q, k, v = (torch.randn(T, H, D, device="cuda").to(torch.bfloat16) for _ in range(3))
    cu = torch.tensor([0, 120, 300], dtype=torch.int32)
    got = ops.attention_varlen_bidirectional(q, k, v, cu, 0.125).float()
    want = ref.attention_varlen_bidirectional(q.float(), k.float(), v.float(), cu, 0.125)
    ops.check_status()
    assert (got - want).abs().max().item() < 0.03


def test_pos_embed_add_and_gelu_erf():
    torch.manual_seed(2)
    T, E, P = 50, 128, 64
    x = torch.randn(T, E, device="cuda").to(torch.bfloat16)
    table = torch.randn(P, E, device="cuda").to(torch.bfloat16)
    idx = torch.randint(0, P, (4, T), device="cuda")
    w = torch.rand(4, T, device="cuda")
    w = w / w.sum(0, keepdim=True)
    want = ref.vision_pos_embed_add(x.float(), table.float(), idx, w)
    got = ops.vision_pos_embed_add(x.clone(), table, idx, w).float()
    assert (got - want).abs().max().item() < 0.05
    y = torch.randn(1000, device="cuda").to(torch.bfloat16)
    torch.testing.assert_close(ops.gelu_erf(y).float(), torch.nn.functional.gelu(y.float()), atol=0.02, rtol=0.02)


def test_qwen3_vl_tiny_gpu_matches_cpu_oracle():
    """The whole model (vision tower, image-token scatter, deepstack, M-RoPE decoder) in bf16 on the
    kernels against the same weights in fp32 through the PyTorch statements of the ops."""
    from mllm_b200.bench_one_batch import make_multimodal_inputs
    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.models.presets import get_preset

    cfg = get_preset("qwen3-vl-tiny")

    def build(device, dtype):
        sc = ServerConfig(model_path="preset:qwen3-vl-tiny", dtype=dtype, max_running_requests=2, max_total_tokens=1024,
                          disable_cuda_graph=True)
        mr = ModelRunner(sc, hf_config=get_preset("qwen3-vl-tiny"), device=device)
        mr.initialize()
        return mr

    gpu, cpu = build("cuda:0", "bfloat16"), build("cpu", "float32")
    sd = {k: v.detach().float().cpu() for k, v in gpu.model.state_dict().items()}
    # both models keep gate/up rows in the same 128-row interleaved layout, so the tensors copy over as they are
    cpu.model.load_state_dict(sd, strict=False)
    image = torch.randint(0, 256, (64, 96, 3), dtype=torch.uint8, generator=torch.Generator().manual_seed(0))
    ids, pix, grid = make_multimodal_inputs(hf_config=cfg, batch_size=1, input_len=40, image=image, seed=0)

    def run(mr):
        dev = mr.device
        L = ids.shape[1]
        slots = mr.req_to_token_pool.alloc(1)
        loc = mr.token_to_kv_pool_allocator.alloc(L)
        sl = torch.tensor(slots, device=dev)
        mr.req_to_token_pool.req_to_token[sl.long(), :L] = loc.view(1, L).int()
        lens = torch.full((1,), L, device=dev, dtype=torch.int32)
        fb = mr.prepare_forward_batch_extend(ids.reshape(-1).to(dev).long(), sl, lens, lens, torch.zeros_like(lens), loc,
                                             extend_seq_lens_cpu=[L], extend_prefix_lens_cpu=[0],
                                             pixel_values=pix.to(dev), image_grid_thw=grid.to(dev))
        return mr.forward(fb).next_token_logits.float().cpu()

    got, want = run(gpu), run(cpu)
    ops.check_status()
    assert (got - want).abs().max().item() < 0.1 * max(1.0, want.abs().max().item())
    assert torch.nn.functional.cosine_similarity(got, want, dim=-1).min().item() > 0.99


def test_vision_tower_graph_replay_equals_eager(monkeypatch):
    """The captured tower (one graph per set of image grids) gives the eager tower's features, for new pixels at
    every replay, for two grids alternating, and after the cache has evicted and re-captured an entry."""
    from mllm_b200.models.presets import get_preset
    from mllm_b200.models.qwen3_vl import Qwen3VLVisionModel

    cfg = get_preset("qwen3-vl-tiny")
    torch.manual_seed(0)
    with torch.device("cuda"):
        vis = Qwen3VLVisionModel(cfg.vision_config, torch.bfloat16)
    for prm in vis.parameters():
        prm.data.normal_(0, 0.05)
    patch_dim = vis.in_channels * vis.temporal_patch_size * vis.patch_size ** 2
    grids = [[[1, 8, 12]], [[1, 4, 4], [1, 8, 8]]]

    def pixels(g, seed):
        n = sum(t * h * w for t, h, w in g)
        return torch.randn(n, patch_dim, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed)).bfloat16()

    monkeypatch.setenv("MLLM_B200_VIT_GRAPH", "0")
    want = {(gi, s): vis(pixels(g, s), g) for gi, g in enumerate(grids) for s in (1, 2)}
    monkeypatch.setenv("MLLM_B200_VIT_GRAPH", "1")
    monkeypatch.setattr(Qwen3VLVisionModel, "_GRAPH_CACHE_ENTRIES", 1)     # every change of grids evicts and re-captures
    for s in (1, 2):
        for gi, g in enumerate(grids):
            got = vis(pixels(g, s), g)
            assert torch.equal(got, want[(gi, s)]), (gi, s)
    assert len(vis.__dict__["_graphs"]) == 1
    ops.check_status()

"""Gated-delta-net kernels against the fp32 PyTorch statements (ragged batches, resumed state)."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def test_rmsnorm_gated():
    torch.manual_seed(0)
    x, g = torch.randn(77, 128, device="cuda").bfloat16(), torch.randn(77, 128, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(128, device="cuda")).bfloat16()
    got = ops.rmsnorm_gated(x, g, w, 1e-6).float()
    want = ref.rmsnorm_gated(x.float(), g.float(), w.float(), 1e-6)
    assert (got - want).abs().max().item() < 0.05


@pytest.mark.parametrize("lens,has", [([5, 1, 300], [0, 1, 0]), ([1, 1, 1, 1], [1, 1, 0, 1]), ([2, 700], [1, 1])])
def test_conv1d_silu_and_state(lens, has):
    torch.manual_seed(1)
    C, K, B = 320, 4, len(lens)
    T = sum(lens)
    x = torch.randn(T, C, device="cuda").bfloat16()
    w = torch.randn(C, K, device="cuda").bfloat16()
    st = torch.randn(B + 2, C, K - 1, device="cuda").bfloat16()
    slots = torch.tensor([b + 1 for b in range(B)], device="cuda", dtype=torch.int32)
    st_ref = st.clone().float().cpu()
    want = ref.causal_conv1d_silu(x.float().cpu(), w.float().cpu(), st_ref, slots.cpu(), lens, has)
    got = ops.causal_conv1d_silu(x, w, st, slots, lens, has)
    assert (got.float().cpu() - want).abs().max().item() < 0.06
    torch.testing.assert_close(st.float().cpu(), st_ref.bfloat16().float())
    ops.check_status()


@pytest.mark.parametrize("lens,has", [([3, 1, 40], [0, 1, 0]), ([1, 1], [1, 0]), ([130], [1])])
def test_gated_delta_rule(lens, has):
    torch.manual_seed(2)
    H, D, B = 4, 128, len(lens)
    T = sum(lens)
    q, k, v = (torch.randn(T, H, D, device="cuda").bfloat16() for _ in range(3))
    g = -torch.rand(T, H, device="cuda") * 0.5
    beta = torch.rand(T, H, device="cuda")
    st = (torch.randn(B + 1, H, D, D, device="cuda") * 0.1).contiguous()
    slots = torch.arange(1, B + 1, device="cuda", dtype=torch.int32)
    st_ref = st.clone().cpu()
    want = ref.gated_delta_rule(q.float().cpu(), k.float().cpu(), v.float().cpu(), g.cpu(), beta.cpu(), st_ref, slots.cpu(), lens, has)
    got = ops.gated_delta_rule(q, k, v, g, beta, st, slots, lens, has)
    ops.check_status()
    scale = want.abs().max().item()
    assert (got.float().cpu() - want).abs().max().item() < 0.02 * scale + 0.02
    assert (st.cpu() - st_ref).abs().max().item() < 0.02 * st_ref.abs().max().item() + 0.02


@pytest.mark.parametrize("lens,has", [([64], [0]), ([1, 63, 65], [1, 0, 1]), ([130, 7], [1, 0]), ([700, 300, 1024], [0, 1, 0]),
                                      ([200] * 5, [1] * 5)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gated_delta_rule_chunk_kernel(lens, has, dtype):
    """The chunk-parallel kernel (64 tokens at a time, tensor-core products) against the fp32 token loop: whole
    chunks, ragged tails, several chunks with the state carried between them, resumed states, both block widths."""
    torch.manual_seed(3)
    H, D, B = 4, 128, len(lens)
    T = sum(lens)
    q, k, v = (torch.randn(T, H, D, device="cuda").to(dtype) for _ in range(3))
    g = -torch.rand(T, H, device="cuda") * 0.5
    beta = torch.rand(T, H, device="cuda")
    st = (torch.randn(B + 1, H, D, D, device="cuda") * 0.1).contiguous()
    slots = torch.arange(1, B + 1, device="cuda", dtype=torch.int32)
    st_ref = st.clone().cpu()
    want = ref.gated_delta_rule(q.float().cpu(), k.float().cpu(), v.float().cpu(), g.cpu(), beta.cpu(), st_ref, slots.cpu(), lens, has)
    ops.set_gdn_extend_backend("cuda_chunkwise")
    try:
        n0 = ops.launch_count()
        got = ops.gated_delta_rule(q, k, v, g, beta, st, slots, lens, has)
        ops.check_status()
        assert ops.launch_count() == n0 + 1
    finally:
        ops.set_gdn_extend_backend("auto")
    scale = want.abs().max().item()
    assert (got.float().cpu() - want).abs().max().item() < 0.02 * scale + 0.02
    assert (st.cpu() - st_ref).abs().max().item() < 0.02 * st_ref.abs().max().item() + 0.02
    assert torch.equal(st[0].cpu(), st_ref[0])            # a state row of no request is left alone


def test_chunk_kernel_wide_value_blocks():
    """Enough (request, head) pairs to fill the GPU: the kernel then takes value blocks of 64 features."""
    torch.manual_seed(5)
    H, D, lens, has = 16, 128, [70, 130, 64, 1, 200], [1, 0, 1, 1, 0]
    B, T = len(lens), sum(lens)
    q, k, v = (torch.randn(T, H, D, device="cuda").bfloat16() for _ in range(3))
    g = -torch.rand(T, H, device="cuda") * 0.5
    beta = torch.rand(T, H, device="cuda")
    st = (torch.randn(B, H, D, D, device="cuda") * 0.1).contiguous()
    slots = torch.arange(B, device="cuda", dtype=torch.int32)
    st_ref = st.clone().cpu()
    want = ref.gated_delta_rule(q.float().cpu(), k.float().cpu(), v.float().cpu(), g.cpu(), beta.cpu(), st_ref, slots.cpu(), lens, has)
    ops.set_gdn_extend_backend("cuda_chunkwise")
    try:
        got = ops.gated_delta_rule(q, k, v, g, beta, st, slots, lens, has)
        ops.check_status()
    finally:
        ops.set_gdn_extend_backend("auto")
    assert (got.float().cpu() - want).abs().max().item() < 0.02 * want.abs().max().item() + 0.02
    assert (st.cpu() - st_ref).abs().max().item() < 0.02 * st_ref.abs().max().item() + 0.02


def test_chunk_and_sequential_kernels_agree_on_a_long_prefill():
    torch.manual_seed(4)
    H, D, lens = 16, 128, [2048, 1500]
    T = sum(lens)
    q, k, v = (torch.randn(T, H, D, device="cuda").bfloat16() for _ in range(3))
    g = -torch.rand(T, H, device="cuda") * 0.3
    beta = torch.rand(T, H, device="cuda")
    slots = torch.tensor([0, 1], device="cuda", dtype=torch.int32)
    outs, states = [], []
    for name in ("cuda_chunkwise", "mllm_kernel"):
        st = torch.zeros(2, H, D, D, device="cuda")
        ops.set_gdn_extend_backend(name)
        try:
            outs.append(ops.gated_delta_rule(q, k, v, g, beta, st, slots, lens, [0, 0]).float())
        finally:
            ops.set_gdn_extend_backend("auto")
        states.append(st)
    ops.check_status()
    assert (outs[0] - outs[1]).abs().max().item() < 0.02 * outs[1].abs().max().item() + 0.02
    assert (states[0] - states[1]).abs().max().item() < 0.02 * states[1].abs().max().item() + 0.02


def test_qwen3_5_tiny_gpu_matches_cpu_oracle():
    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.models.presets import get_preset

    def build(device, dtype):
        sc = ServerConfig(model_path="preset:qwen3.5-tiny", dtype=dtype, max_running_requests=2, max_total_tokens=1024,
                          disable_cuda_graph=True)
        mr = ModelRunner(sc, hf_config=get_preset("qwen3.5-tiny"), device=device)
        mr.initialize()
        return mr

    gpu, cpu = build("cuda:0", "bfloat16"), build("cpu", "float32")
    cpu.model.load_state_dict({k: v.detach().float().cpu() for k, v in gpu.model.state_dict().items()}, strict=False)
    cpu.model.post_load()
    ids = torch.randint(0, 1000, (2, 20), generator=torch.Generator().manual_seed(0))

    def run(mr):
        dev = mr.device
        B, L = ids.shape
        slots = mr.req_to_token_pool.alloc(B)
        loc = mr.token_to_kv_pool_allocator.alloc(B * L)
        sl = torch.tensor(slots, device=dev)
        mr.req_to_token_pool.req_to_token[sl.long(), :L] = loc.view(B, L).int()
        lens = torch.full((B,), L, device=dev, dtype=torch.int32)
        fb = mr.prepare_forward_batch_extend(ids.reshape(-1).to(dev).long(), sl, lens, lens, torch.zeros_like(lens), loc,
                                             extend_seq_lens_cpu=[L] * B, extend_prefix_lens_cpu=[0] * B)
        outs = [mr.forward(fb).next_token_logits.float().cpu()]
        nxt = outs[-1].argmax(-1).to(dev)
        loc1 = mr.token_to_kv_pool_allocator.alloc(B)
        mr.req_to_token_pool.req_to_token[sl.long(), L] = loc1.int()
        fbd = mr.prepare_forward_batch_decode(nxt, sl, torch.full((B,), L + 1, device=dev, dtype=torch.int32), loc1, max_seq_len=L + 1)
        outs.append(mr.forward(fbd).next_token_logits.float().cpu())
        return torch.stack(outs)

    got, want = run(gpu), run(cpu)
    ops.check_status()
    assert torch.nn.functional.cosine_similarity(got.flatten(0, 1), want.flatten(0, 1), dim=-1).min().item() > 0.99

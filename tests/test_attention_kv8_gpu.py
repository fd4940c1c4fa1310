"""An 8-bit KV cache (unscaled e4m3 / e5m2) on the package's kernels: K and V rounded on the way in by the cache-write
kernel and by the fused q/k prologue, and read by the single-role tcgen05 attention kernel, which widens a tile on
its way into shared memory -- prefill and decode at head sizes 64, 128 and 256, against the fp32 statement over
the same 8-bit cache; then a model with such a cache under CUDA graphs against the CPU model."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def _err(a, b):
    return (a.float() - b.float()).abs().max().item()


def _setup(D, fmt, seq_lens, prefix_lens, hq, hkv, dtype=torch.bfloat16, seed=0, head_major=False):
    torch.manual_seed(seed)
    B = len(seq_lens)
    ctx = max(seq_lens) + 8
    total = sum(seq_lens)
    slots = total + 64
    shape = (hkv, slots, D) if head_major else (slots, hkv, D)
    kc, vc = (torch.randn(shape, device=DEV, dtype=dtype).to(FP8[fmt]) for _ in range(2))
    if head_major:
        kc, vc = kc.transpose(0, 1), vc.transpose(0, 1)
    rtt = torch.zeros(B + 3, ctx, dtype=torch.int32, device=DEV)
    perm = torch.randperm(slots - 1, device=DEV)[:total].int() + 1
    req = torch.arange(B, device=DEV, dtype=torch.int32) + 2
    off = 0
    for b, s in enumerate(seq_lens):
        rtt[req[b], :s] = perm[off:off + s]
        off += s
    ext = [s - p for s, p in zip(seq_lens, prefix_lens)]
    q = torch.randn(sum(ext), hq, D, device=DEV, dtype=dtype)
    q_start = torch.tensor([sum(ext[:i]) for i in range(B)], dtype=torch.int32, device=DEV)
    return dict(q=q, kc=kc, vc=vc, rtt=rtt, req=req, seq=torch.tensor(seq_lens, dtype=torch.int32, device=DEV),
                pre=torch.tensor(prefix_lens, dtype=torch.int32, device=DEV), q_start=q_start, max_q=max(ext))


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_cache_write_rounds_like_a_cast(fmt, dtype):
    torch.manual_seed(0)
    hkv, D, slots, T = 4, 128, 300, 77
    for head_major in (False, True):
        shape = (hkv, slots, D) if head_major else (slots, hkv, D)
        kc, vc = (torch.zeros(shape, device=DEV, dtype=FP8[fmt]) for _ in range(2))
        if head_major:
            kc, vc = kc.transpose(0, 1), vc.transpose(0, 1)
        k = torch.randn(T, hkv * D, device=DEV, dtype=dtype) * 3
        v = torch.randn(T, hkv * D, device=DEV, dtype=dtype) * 3
        loc = torch.randperm(slots, device=DEV)[:T]
        n0 = ops.launch_count()
        ops.kv_write(k, v, loc, kc, vc)
        ops.check_status()
        assert ops.launch_count() > n0
        assert torch.equal(kc[loc].view(torch.uint8), k.view(T, hkv, D).to(FP8[fmt]).view(torch.uint8))
        assert torch.equal(vc[loc].view(torch.uint8), v.view(T, hkv, D).to(FP8[fmt]).view(torch.uint8))


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_fused_prologue_writes_the_8_bit_cache(fmt):
    torch.manual_seed(1)
    hq, hkv, D, slots, T = 8, 2, 128, 400, 90
    qkv = torch.randn(T, (hq + 2 * hkv) * D, device=DEV, dtype=torch.bfloat16)
    qw, kw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16(), (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    pos = torch.arange(T, device=DEV) + 5
    loc = torch.randperm(slots, device=DEV)[:T]
    caches = [torch.zeros(hkv, slots, D, device=DEV, dtype=FP8[fmt]).transpose(0, 1) for _ in range(4)]
    a, b = qkv.clone(), qkv.clone()
    n0 = ops.launch_count()
    ops.qk_norm_rope_kv_write(a, qw, kw, pos, loc, caches[0], caches[1], hq, hkv, D, 1e6, 1e-6)
    ops.check_status()
    assert ops.launch_count() > n0
    ref.qk_norm_rope_kv_write(b, qw, kw, pos, loc, caches[2], caches[3], hq, hkv, D, 1e6, 1e-6)
    assert _err(a[:, : (hq + hkv) * D], b[:, : (hq + hkv) * D]) < 3e-2
    # V is copied: the bytes agree; K went through sines and cosines computed twice: a last-place difference in 16
    # bits can move an 8-bit value to its neighbour, rarely
    assert torch.equal(caches[1][loc].view(torch.uint8), caches[3][loc].view(torch.uint8))
    kd, kr = caches[0][loc].float(), caches[2][loc].float()
    assert (kd != kr).float().mean().item() < 0.02
    assert ((kd - kr).abs() <= 0.26 * kr.abs() + 1e-3).all()


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("seq_lens,prefix_lens", [([3], [0]), ([65], [0]), ([700, 33], [0, 0]), ([200, 130], [64, 1]),
                                                  ([1000], [873])])
def test_prefill(fmt, D, seq_lens, prefix_lens):
    s = _setup(D, fmt, seq_lens, prefix_lens, 8, 2, head_major=D == 128)
    scale = D ** -0.5
    n0 = ops.launch_count()
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"])
    ops.check_status()
    assert ops.launch_count() > n0
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("seq_lens", [[1], [64], [65], [2048], [1, 700, 64, 129]])
def test_decode(fmt, D, seq_lens):
    s = _setup(D, fmt, seq_lens, [x - 1 for x in seq_lens], 32, 8, dtype=torch.float16 if D == 64 else torch.bfloat16,
               seed=1, head_major=True)
    scale = D ** -0.5
    n0 = ops.launch_count()
    got = ops.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale, max_seq_len=max(seq_lens))
    ops.check_status()
    assert ops.launch_count() > n0
    want = ref.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale)
    assert _err(got, want) < 3e-2


def test_window_and_soft_cap_over_an_8_bit_cache():
    D = 128
    s = _setup(D, "e4m3", [700, 300], [0, 100], 8, 4, seed=4)
    scale = D ** -0.5 * 3.0
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"], window=100, logit_cap=20.0)
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                 window=100, logit_cap=20.0)
    assert _err(got, want) < 3e-2


def test_model_with_an_8_bit_cache_under_cuda_graphs():
    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.models.presets import get_preset

    def build(device, dtype, kv):
        sc = ServerConfig(model_path="preset:qwen3-tiny", dtype=dtype, max_running_requests=2, max_total_tokens=1024)
        mr = ModelRunner(sc, hf_config=get_preset("qwen3-tiny"), kv_cache_dtype=kv, device=device)
        mr.initialize()
        return mr

    gpu, cpu = build("cuda:0", "bfloat16", "fp8_e4m3"), build("cpu", "float32", "auto")
    assert gpu.token_to_kv_pool.store.dtype == torch.float8_e4m3fn and gpu.cuda_graph_runner is not None
    cpu.model.load_state_dict({k: v.detach().float().cpu() for k, v in gpu.model.state_dict().items()}, strict=False)
    if hasattr(cpu.model, "post_load"):
        cpu.model.post_load()
    ids = torch.randint(0, 1000, (2, 24), generator=torch.Generator().manual_seed(1))

    def run(mr):
        dev = mr.device
        B, L = ids.shape
        slots = mr.req_to_token_pool.alloc(B)
        loc = mr.token_to_kv_pool_allocator.alloc(B * L).view(B, L)
        sl = torch.tensor(slots, device=dev)
        mr.req_to_token_pool.req_to_token[sl.long(), :L] = loc.int()
        full = lambda n: torch.full((B,), n, device=dev, dtype=torch.int32)  # noqa: E731
        fb = mr.prepare_forward_batch_extend(ids.reshape(-1).to(dev).long(), sl, full(L), full(L), full(0), loc.reshape(-1),
                                             extend_seq_lens_cpu=[L] * B, extend_prefix_lens_cpu=[0] * B)
        outs = [mr.forward(fb).next_token_logits.float().cpu()]
        nxt = ids[:, -1].to(dev)                       # the same forced tokens on both sides
        for step in range(2):
            loc1 = mr.token_to_kv_pool_allocator.alloc(B)
            mr.req_to_token_pool.req_to_token[sl.long(), L + step] = loc1.int()
            fbd = mr.prepare_forward_batch_decode(nxt, sl, full(L + step + 1), loc1, max_seq_len=L + step + 1)
            outs.append(mr.forward(fbd).next_token_logits.float().cpu())
            nxt = ids[:, step].to(dev)
        return torch.stack(outs)

    got, want = run(gpu), run(cpu)
    ops.check_status()
    cos = torch.nn.functional.cosine_similarity(got.flatten(0, 1), want.flatten(0, 1), dim=-1)
    assert cos.min().item() > 0.97, cos

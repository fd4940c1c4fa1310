"""Model configurations off the main path of the attention kernels on a GPU: head sizes 64 and 256 (the
single-role tcgen05 kernel; the fused q/k prologue is written for head size 128, so norms, rotation and the cache
write run as separate steps), a sliding window, and an 8-bit KV cache (attention on the library / batched PyTorch
fallbacks).  Each case compares the GPU model (bf16) with the CPU model (fp32) holding the same weights: prefill
in two chunks, then decode."""
import pytest
import torch

from mllm_b200 import ops

pytestmark = pytest.mark.gpu


def _pair(preset, kv="auto", **overrides):
    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.models.presets import get_preset

    def build(device, dtype, kv_dtype):
        sc = ServerConfig(model_path=f"preset:{preset}", dtype=dtype, max_running_requests=2, max_total_tokens=1024,
                          disable_cuda_graph=True)
        mr = ModelRunner(sc, hf_config=get_preset(preset, **overrides), kv_cache_dtype=kv_dtype, device=device)
        mr.initialize()
        return mr

    gpu, cpu = build("cuda:0", "bfloat16", kv), build("cpu", "float32", "auto")
    cpu.model.load_state_dict({k: v.detach().float().cpu() for k, v in gpu.model.state_dict().items()}, strict=False)
    if hasattr(cpu.model, "post_load"):
        cpu.model.post_load()
    return gpu, cpu


def _run(mr, ids):
    dev = mr.device
    B, L = ids.shape
    half = L // 2
    slots = mr.req_to_token_pool.alloc(B)
    loc = mr.token_to_kv_pool_allocator.alloc(B * L).view(B, L)
    sl = torch.tensor(slots, device=dev)
    mr.req_to_token_pool.req_to_token[sl.long(), :L] = loc.int()
    full = lambda n: torch.full((B,), n, device=dev, dtype=torch.int32)  # noqa: E731
    fb = mr.prepare_forward_batch_extend(ids[:, :half].reshape(-1).to(dev).long(), sl, full(half), full(half), full(0),
                                         loc[:, :half].reshape(-1), extend_seq_lens_cpu=[half] * B, extend_prefix_lens_cpu=[0] * B)
    mr.forward(fb)
    fb = mr.prepare_forward_batch_extend(ids[:, half:].reshape(-1).to(dev).long(), sl, full(L), full(L - half), full(half),
                                         loc[:, half:].reshape(-1), extend_seq_lens_cpu=[L - half] * B,
                                         extend_prefix_lens_cpu=[half] * B)
    outs = [mr.forward(fb).next_token_logits.float().cpu()]
    nxt = outs[-1].argmax(-1).to(dev)
    loc1 = mr.token_to_kv_pool_allocator.alloc(B)
    mr.req_to_token_pool.req_to_token[sl.long(), L] = loc1.int()
    fbd = mr.prepare_forward_batch_decode(nxt, sl, full(L + 1), loc1, max_seq_len=L + 1)
    outs.append(mr.forward(fbd).next_token_logits.float().cpu())
    return torch.stack(outs)


def _close(got, want, floor=0.985):
    cos = torch.nn.functional.cosine_similarity(got.flatten(0, 1), want.flatten(0, 1), dim=-1)
    assert cos.min().item() > floor, cos


@pytest.mark.parametrize("preset,overrides", [
    ("llama-tiny", dict(head_dim=64, num_attention_heads=4, num_key_value_heads=2)),       # head size 64
    ("llama-tiny", dict(sliding_window=8, architectures=["MistralForCausalLM"])),          # sliding window
    ("qwen2-tiny", dict(head_dim=64)),                                                     # q/k/v biases + head size 64
    ("qwen3.5-tiny", dict(head_dim=256)),                                                  # hybrid model, published head size
])
def test_gpu_model_off_the_main_attention_path_matches_cpu(preset, overrides):
    gpu, cpu = _pair(preset, **overrides)
    ids = torch.randint(0, 1000, (2, 24), generator=torch.Generator().manual_seed(0))
    got, want = _run(gpu, ids), _run(cpu, ids)
    ops.check_status()
    _close(got, want)


def test_fp8_kv_cache_on_gpu_stays_close_to_the_cpu_model():
    gpu, cpu = _pair("qwen3-tiny", kv="fp8_e4m3")
    assert gpu.token_to_kv_pool.store.dtype == torch.float8_e4m3fn and gpu.cuda_graph_runner is None
    ids = torch.randint(0, 1000, (2, 24), generator=torch.Generator().manual_seed(1))
    got, want = _run(gpu, ids), _run(cpu, ids)
    ops.check_status()
    _close(got, want, floor=0.97)


def test_bounded_flag_wait_runs_out_into_a_status_and_the_context_stays_usable():
    """Failure detection without a fault: a kernel waits (with its built-in bound) on a flag that nothing
    sets; it gives up, records the status word, and returns.  The host reads the status as an error, the
    word is cleared by the read, and the device keeps working."""
    import time

    from mllm_b200.ops import reference as ref

    ops.check_status()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    assert ops.ext().tp_wait_flags(flags, 1, 1) == 0          # launches fine; nobody will ever write epoch 1
    with pytest.raises(RuntimeError, match="peer flag wait timed out"):
        ops.check_status()
    assert time.perf_counter() - t0 < 30.0                    # bounded: seconds, not forever
    ops.check_status()                                        # cleared by the read above
    flags.fill_(3)
    assert ops.ext().tp_wait_flags(flags, 8, 3) == 0          # a wait that is satisfied leaves no status
    ops.check_status()
    x = torch.randn(16, 256, device="cuda").bfloat16()
    w = torch.ones(256, device="cuda").bfloat16()
    got = ops.rmsnorm(x, w, 1e-6).float()
    assert (got - ref.rmsnorm(x.float(), w.float(), 1e-6)).abs().max().item() < 0.05

"""``--<section>.<field>`` command line and ServerConfig validation (reference cases:
pymllm/tests/test_bench_one_batch.py:30-150)."""
import pytest

from mllm_b200.configs import GlobalConfig, ServerConfig, make_args, read_args


@pytest.fixture(autouse=True)
def _fresh():
    GlobalConfig.reset()
    yield
    GlobalConfig.reset()


def test_defaults_untouched_when_not_typed():
    cfg = read_args([])
    assert cfg.server.port == 30000 and cfg.server.max_running_requests == 1
    assert cfg.server.tp_size == 1 and cfg.quantization.method is None


def test_scalar_bool_and_literal_options():
    cfg = read_args(["--server.model_path", "/m", "--server.port", "8080", "--server.disable_cuda_graph",
                     "--server.sleep_on_idle", "false", "--server.dtype", "bfloat16", "--server.tp_size", "8",
                     "--quantization.method", "compressed-tensors", "--quantization.kv_cache_dtype", "bfloat16"])
    s = cfg.server
    assert str(s.model_path) == "/m" and str(s.tokenizer_path) == "/m" and s.port == 8080
    assert s.disable_cuda_graph is True and s.sleep_on_idle is False and s.dtype == "bfloat16" and s.tp_size == 8
    assert cfg.quantization.method == "compressed-tensors" and str(cfg.model.model_path) == "/m"


def test_model_path_sync_other_direction():
    cfg = read_args(["--model.model_path", "/x"]) if any(
        a.dest == "model__model_path" for a in make_args()._actions) else None
    if cfg is not None:
        assert str(cfg.server.model_path) == "/x"


def test_bad_choice_rejected():
    with pytest.raises(SystemExit):
        read_args(["--server.dtype", "int3"])


def test_bad_bool_rejected():
    with pytest.raises(SystemExit):
        read_args(["--server.disable_cuda_graph", "maybe"])


@pytest.mark.parametrize("kw", [dict(port=0), dict(stream_interval=0), dict(mem_fraction_static=1.5),
                                dict(max_running_requests=0), dict(radix_cache_page_size=0),
                                dict(tensor_transport_mode="bogus"), dict(tensor_transport_mode="cuda_ipc"),
                                dict(tp_size=3), dict(max_queued_requests=-1)])
def test_validation(kw):
    with pytest.raises(ValueError):
        ServerConfig(model_path=None, **kw)


def test_page_size_alias():
    assert ServerConfig(page_size=64).radix_cache_page_size == 64
    cfg = read_args(["--server.radix_cache_page_size", "16"])
    assert cfg.server.page_size == 16


def test_revalidation_on_cli():
    with pytest.raises(ValueError):
        read_args(["--server.port", "70000"])


def test_kv_pool_capacity_from_the_memory_profile(monkeypatch):
    """Token capacity = (free after load - (1 - mem_fraction_static) x free before load) / bytes per token,
    capped by max_total_tokens; too little memory raises with the knob named in the message."""
    import pytest
    import torch

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import model_runner as mrmod
    from mllm_b200.executor import ModelRunner

    mr = ModelRunner(ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=2,
                                  max_total_tokens=None, mem_fraction_static=0.8), device="cpu")
    mr.initialize()
    cell = mr.cell_bytes()
    assert cell == 2 * mr.num_hidden_layers * mr.num_kv_heads * mr.head_dim * 4          # K and V, fp32
    mr._pre_load_avail_gib = 100.0
    monkeypatch.setattr(mrmod, "get_available_gpu_memory", lambda *_a, **_k: 80.0)
    prof = mr._profile_max_num_tokens()
    assert prof.rest_gib == pytest.approx(80.0 - 100.0 * 0.2)
    assert prof.max_total_num_tokens == int(60.0 * (1 << 30) // cell) and prof.cell_bytes == cell
    mr.server_config.max_total_tokens = 4096
    mr.init_memory_pool()
    assert mr.max_total_num_tokens == 4096 and mr.req_to_token_pool.size == 2 + 8
    monkeypatch.setattr(mrmod, "get_available_gpu_memory", lambda *_a, **_k: 10.0)
    with pytest.raises(RuntimeError, match="mem_fraction_static"):
        mr.init_memory_pool()


def test_hybrid_state_pool_is_allocated_before_the_kv_pool_is_sized():
    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner

    order = []
    mr = ModelRunner(ServerConfig(model_path="preset:qwen3.5-tiny", dtype="float32", max_running_requests=3,
                                  max_total_tokens=512, enable_mamba_cache=True, mamba_cache_slots=5), device="cpu")
    for name in ("_init_state_pool", "init_memory_pool"):
        orig = getattr(mr, name)
        setattr(mr, name, (lambda o, n: lambda: (order.append(n), o())[1])(orig, name))
    mr.initialize()
    assert order == ["_init_state_pool", "init_memory_pool"]
    # one state row per request-table row, the spare padding row included
    assert mr.gdn_pool.slots == mr.req_to_token_pool.size + 1 == 3 + 8 + 1 and mr.gdn_pool.track_slots == 5


def test_fp8_kv_cache_halves_the_cache_and_stays_close():
    """``kv_cache_dtype fp8_e4m3``: one byte per cached value, logits close to the 16-/32-bit cache run
    (prefill in two chunks so that cached keys are really read back, then a decode step)."""
    import torch

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner

    def run(kv):
        mr = ModelRunner(ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=2,
                                      max_total_tokens=256), kv_cache_dtype=kv, device="cpu")
        mr.initialize()
        ids = (torch.arange(20) * 13) % 1000
        slots = mr.req_to_token_pool.alloc(1)
        sl = torch.tensor(slots)
        loc = mr.token_to_kv_pool_allocator.alloc(20)
        mr.req_to_token_pool.req_to_token[slots[0], :20] = loc.int()
        mr.forward(mr.prepare_forward_batch_extend(ids[:12], sl, torch.tensor([12]), torch.tensor([12]), torch.tensor([0]), loc[:12]))
        out = mr.forward(mr.prepare_forward_batch_extend(ids[12:], sl, torch.tensor([20]), torch.tensor([8]), torch.tensor([12]), loc[12:]))
        logits = [out.next_token_logits]
        loc1 = mr.token_to_kv_pool_allocator.alloc(1)
        mr.req_to_token_pool.req_to_token[slots[0], 20] = loc1.int()
        logits.append(mr.forward(mr.prepare_forward_batch_decode(logits[0].argmax(-1), sl, torch.tensor([21]), loc1)).next_token_logits)
        return torch.cat(logits), mr

    ref_logits, mr_ref = run("auto")
    fp8_logits, mr_fp8 = run("fp8_e4m3")
    assert mr_fp8.token_to_kv_pool.store.dtype == torch.float8_e4m3fn
    assert mr_fp8.cell_bytes() * 4 == mr_ref.cell_bytes()                 # fp32 reference run vs one byte
    err = (fp8_logits - ref_logits).abs().max().item()
    assert 0 < err < 0.05 * ref_logits.abs().max().item() + 0.02
    assert torch.equal(fp8_logits.argmax(-1), ref_logits.argmax(-1))


def test_helper_command_lists_architectures_and_extensions(capsys):
    import json

    from mllm_b200.__main__ import main

    main(["show-config"])
    info = json.loads(capsys.readouterr().out)
    assert "Qwen3ForCausalLM" in info["architectures"] and "compressed-tensors" in info["quantization"]
    assert set(info["extensions"]) == {"mllm_b200_C", "mllm_b200_host"}
    main(["models"])
    assert "Qwen3VLForConditionalGeneration" in capsys.readouterr().out.split()

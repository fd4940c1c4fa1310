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

"""The multi-process engine (tokenizer -> scheduler -> detokenizer over ZMQ) on CPU, including the
liveness path: a worker process that dies turns the engine unhealthy (host-side fault, no GPU)."""
import time

import pytest

from mllm_b200.configs import ServerConfig
from mllm_b200.engine.launch import Engine


def _cfg():
    return ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=4, max_total_tokens=1024,
                        context_length=128, log_level="warning")


def test_multiproc_generate_matches_inproc_and_detects_dead_worker():
    ref = Engine(_cfg(), mode="inproc", device="cpu").launch()
    want = ref.generate("hello", {"max_new_tokens": 5, "temperature": 0.0})["output_ids"]
    ref.shutdown()
    eng = Engine(_cfg(), mode="multiproc", device="cpu").launch()
    try:
        got = eng.generate("hello", {"max_new_tokens": 5, "temperature": 0.0}, timeout=120)
        assert got["output_ids"] == want and got["meta_info"]["finish_reason"] == "length"
        chunks = list(eng.generate("hello", {"max_new_tokens": 5, "temperature": 0.0}, stream=True))
        assert chunks[-1]["output_ids"] == want
        # host-side failure injection: kill the detokenizer process
        eng._procs[2].terminate()
        eng._procs[2].join(10)
        eng._health_loop.__func__  # the monitor thread polls every 5 s
        deadline = time.time() + 12
        while eng.is_healthy and time.time() < deadline:
            time.sleep(0.25)
        assert not eng.is_healthy
        with pytest.raises((RuntimeError, TimeoutError)):
            eng.generate("x", {"max_new_tokens": 2}, timeout=5)
    finally:
        eng.shutdown()

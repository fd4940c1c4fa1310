"""bench_one_batch CLI / JSONL schema and bench_serve workload + report on CPU."""
import asyncio
import json

import pytest

from mllm_b200 import bench_one_batch as bob
from mllm_b200 import bench_serve as bs
from mllm_b200.configs import GlobalConfig, ServerConfig
from mllm_b200.engine.launch import Engine


@pytest.fixture(autouse=True)
def _fresh():
    GlobalConfig.reset()
    yield
    GlobalConfig.reset()


def test_bench_one_batch_cli_and_settings():
    cfg, args = bob.parse_args(["--server.model_path", "preset:qwen3-tiny", "--batch-size", "1", "4", "--input-len", "16",
                                "--output-len", "8", "--seed", "7", "--server.tp_size", "1"])
    assert args.batch_size == [1, 4] and args.input_len == [16] and args.input_len_was_provided and args.seed == 7
    assert [(s.batch_size, s.input_len, s.output_len) for s in bob.generate_settings(args)] == [(1, 16, 8), (4, 16, 8)]
    _, a2 = bob.parse_args(["--image", "x.png"])
    assert bob.generate_settings(a2)[0].input_len == 0
    with pytest.raises(SystemExit):
        bob.parse_args(["--batch-size", "0"])
    ids = bob.make_synthetic_input_ids(batch_size=2, input_len=5, vocab_size=151936, seed=1)
    assert ids.shape == (2, 5) and int(ids.max()) < 10000
    assert bob.make_synthetic_input_ids(batch_size=2, input_len=5, vocab_size=151936, seed=1).equal(ids)


def test_bench_one_batch_jsonl_schema(tmp_path):
    out = tmp_path / "r.jsonl"
    cfg, args = bob.parse_args(["--server.model_path", "preset:qwen3-tiny", "--server.dtype", "float32",
                                "--server.max_total_tokens", "2048", "--batch-size", "2", "--input-len", "16",
                                "--output-len", "4", "--result-filename", str(out)])
    rows = bob.run_benchmark(cfg, args)
    row = json.loads(out.read_text().strip())
    for k in ("run_name", "batch_size", "input_len", "output_len", "prefill_latency", "prefill_throughput",
              "median_decode_latency", "median_decode_throughput", "total_latency", "overall_throughput"):
        assert k in row
    assert row["batch_size"] == 2 and rows[0]["overall_throughput"] > 0
    assert cfg.server.max_running_requests >= 2  # raised to cover the batch


def test_bench_one_batch_profile_writes_a_trace_per_stage(tmp_path, monkeypatch):
    """``--profile`` with the CPU activity: one trace file for the prefill, one for the decode window."""
    import os

    monkeypatch.setenv("MLLM_B200_PROFILE_DIR", str(tmp_path / "traces"))
    cfg, args = bob.parse_args(["--server.model_path", "preset:qwen3-tiny", "--server.dtype", "float32",
                                "--server.max_total_tokens", "2048", "--batch-size", "2", "--input-len", "16",
                                "--output-len", "6", "--skip-warmup", "--profile", "--profile-activities", "CPU",
                                "--profile-start-step", "1", "--profile-steps", "2",
                                "--result-filename", str(tmp_path / "r.jsonl")])
    rows = bob.run_benchmark(cfg, args)
    traces = rows[0]["profile_traces"]
    assert len(traces) == 2 and "_prefill_" in traces[0] and "_decode_" in traces[1]
    assert all(os.path.getsize(t) > 0 for t in traces)
    cfg, args = bob.parse_args(["--server.model_path", "preset:qwen3-tiny", "--server.dtype", "float32",
                                "--server.max_total_tokens", "2048", "--batch-size", "1", "--input-len", "8",
                                "--output-len", "3", "--skip-warmup", "--profile", "--profile-activities", "CPU",
                                "--profile-stage", "decode", "--result-filename", str(tmp_path / "r2.jsonl")])
    assert len(bob.run_benchmark(cfg, args)[0]["profile_traces"]) == 1


def test_bench_one_batch_skips_oversize(tmp_path):
    cfg, args = bob.parse_args(["--server.model_path", "preset:qwen3-tiny", "--server.dtype", "float32",
                                "--server.max_total_tokens", "64", "--batch-size", "8", "--input-len", "64", "--output-len", "4",
                                "--skip-warmup", "--result-filename", str(tmp_path / "r.jsonl")])
    assert bob.run_benchmark(cfg, args) == []


def test_bench_serve_workload_and_poisson_run():
    work = bs.make_workload(40, (8, 40), (2, 6), 0.5, 16, 1000, seed=3)
    assert work == bs.make_workload(40, (8, 40), (2, 6), 0.5, 16, 1000, seed=3)
    shared = [w for w in work if len(w[0]) > 16 and w[0][:16] == work[0][0][:16] or w[0][:16] == [x for x in w[0][:16]]]
    arr = bs.poisson_arrivals(40, 200.0, 3)
    assert arr[0] == 0.0 and all(b >= a for a, b in zip(arr, arr[1:]))
    assert bs.percentile([1, 2, 3, 4], 50) == 2.5
    sc = ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=8, max_total_tokens=4096,
                      context_length=128, log_level="warning", chunked_prefill_size=64)
    eng = Engine(sc, mode="inproc", device="cpu").launch()
    try:
        rep = asyncio.run(bs.run_poisson(work, arr, engine=eng))
        assert rep["completed"] == 40 and rep["failed"] == 0 and rep["ttft_ms"]["p50"] > 0
        assert rep["total_output_tokens"] == sum(w[1] for w in work) and rep["cached_token_ratio"] > 0.0
        rows = asyncio.run(bs.run_sequential([8, 16], 4, 1, 1000, 0, engine=eng))
        assert [r["pp"] for r in rows] == [8, 16] and all(r["decode_tok_s"] > 0 for r in rows)
    finally:
        eng.shutdown()


def test_random_checkpoint_directory_loads_here_and_in_transformers(tmp_path):
    """The seeded random-init checkpoint the benchmark's reference arm serves: a plain HF directory
    (config.json + safetensors + index) that our runner and transformers both load, with the same logits."""
    import torch

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.io.random_checkpoint import write_random_checkpoint

    tr = pytest.importorskip("transformers")
    d = write_random_checkpoint("qwen3-tiny", tmp_path / "ck", seed=0, dtype=torch.float32, device="cpu")
    assert (d / ".complete").exists() and write_random_checkpoint("qwen3-tiny", d) == d      # second call reuses it
    mr = ModelRunner(ServerConfig(model_path=str(d), dtype="float32", max_running_requests=2, max_total_tokens=256), device="cpu")
    mr.initialize()
    ids = torch.arange(9).view(1, 9) * 5 % 1000
    slots = mr.req_to_token_pool.alloc(1)
    loc = mr.token_to_kv_pool_allocator.alloc(9)
    mr.req_to_token_pool.req_to_token[slots[0], :9] = loc.int()
    lens = torch.tensor([9])
    got = mr.forward(mr.prepare_forward_batch_extend(ids[0], torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)).next_token_logits
    hf = tr.AutoModelForCausalLM.from_pretrained(str(d), torch_dtype=torch.float32).eval()
    with torch.no_grad():
        want = hf(ids).logits[:, -1]
    torch.testing.assert_close(got, want, atol=5e-4, rtol=5e-4)

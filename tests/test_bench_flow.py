"""The flagship bench's control flow on the host: single rank, two data-parallel ranks (gloo), and
the watchdog that bounds a run that never finishes."""

import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
TINY = ["--device", "cpu", "--model", "qwen3-tiny", "--batch-size", "2", "--input-len", "32", "--output-len", "4",
        "--steps", "2"]


def _last_json(stdout: str) -> dict:
    lines = [ln for ln in stdout.splitlines() if ln.startswith("{")]
    assert lines, stdout
    return json.loads(lines[-1])


def _free_port() -> str:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def _env() -> dict:
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    return env


def test_single_rank_line_has_the_contract_keys():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), *TINY], capture_output=True, text=True, timeout=300,
                       env=_env(), cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    out = _last_json(p.stdout)
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in out
    assert out["n_gpus"] == 1 and out["warmup"] >= 3 and out["config"]["global_batch"] == 2
    assert out["e2e"]["h2d_bytes_per_step"] == 2 * 32 * 4 and out["e2e"]["d2h_bytes_per_step"] == 4 * 2 * 8
    assert out["value"] > 0 and out["e2e"]["value"] > 0


def test_two_data_parallel_ranks_count_both_batches():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), str(ROOT / "bench.py"), "--gpus", "2", "--parallelism", "dp", *TINY]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=_env(), cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, "exactly one rank prints the result"
    out = json.loads(lines[0])
    assert out["n_gpus"] == 2 and out["scaling"] == "weak"
    assert out["config"]["parallelism"] == "dp2" and out["config"]["global_batch"] == 4
    tokens = 4 * (32 + 4)
    assert abs(out["value"] - tokens / (out["ms_per_step"] / 1e3)) < 1e-6 * out["value"]
    assert out["e2e"]["h2d_bytes_per_step"] == 2 * (2 * 32 * 4)


def test_watchdog_ends_a_run_that_never_finishes():
    code = ("import sys, time; sys.path.insert(0, %r); import bench; "
            "w = bench.Watchdog(0.5, 0, 4); w.log('stuck phase'); time.sleep(30)") % str(ROOT)
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60, env=_env())
    assert p.returncode == 3
    out = _last_json(p.stdout)
    assert out["value"] is None and "stuck phase" in out["error"] and out["n_gpus"] == 4
    assert "time.sleep" in p.stderr or "File" in p.stderr   # the stack dump


def test_two_tensor_parallel_ranks_share_one_batch():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), str(ROOT / "bench.py"), "--gpus", "2", *TINY]       # tensor parallelism is the default layout at N > 1
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=_env(), cwd=ROOT)
    assert p.returncode == 0, p.stderr[-2000:]
    out = _last_json(p.stdout)
    assert out["n_gpus"] == 2 and out["scaling"] == "strong"
    assert out["config"]["parallelism"] == "tp2" and out["config"]["global_batch"] == 2
    assert out["e2e"]["h2d_bytes_per_step"] == 2 * 32 * 4

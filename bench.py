"""Flagship benchmark: Qwen3-8B-shaped decoder, bf16, one batch of `--batch-size` requests with
input_len 2048 and output_len 128 (prefill + 127 greedy decode steps) — the reference's
``bench_one_batch`` workload — on N GPUs of one node with tensor parallelism TP=N.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference --gpus 1 --steps 5 --warmup 3

One *step* is one complete batch: prefill of batch x 2048 seeded random token ids followed by
127 decode steps (128 output tokens per request).  ``value`` is whole-job tokens per second,
``batch * (2048 + 128) / seconds_per_step``, with the step timed on the device by CUDA events
(maximum over ranks).  ``e2e`` repeats the measurement through the public
``BenchRunner.extend`` / ``decode`` API with the prompt ids copied from pinned host memory
and every step's sampled ids read back to the host, timed by the host clock around device
synchronisation.  Weights are random-init (seeded N(0, 0.02)); data are synthetic.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "tokens_per_s_bench_one_batch_in2048_out128"


def parse() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--input-len", type=int, default=2048)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


# --------------------------------------------------------------------------------------------
# clocks: sample nvidia-smi while the timed region runs
# --------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump() -> None:
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # "under load" = samples drawing more than 40 % of the maximum sampled power
        loaded = [s for s, p in zip(sm, power) if power and p > 0.4 * max(power)] or sm
        return {
            "sm_mhz": statistics.median(loaded) if loaded else None,
            "sm_max_mhz": max(mx) if mx else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


# --------------------------------------------------------------------------------------------
# our implementation
# --------------------------------------------------------------------------------------------
def run_ours(a: argparse.Namespace) -> dict:
    import torch
    import torch.distributed as dist

    from mllm_b200 import ops
    from mllm_b200.bench_one_batch import BenchRunner, make_synthetic_input_ids
    from mllm_b200.configs import GlobalConfig
    from mllm_b200.parallel import state as pstate

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {a.gpus}")
    torch.cuda.set_device(local_rank)

    GlobalConfig.reset()
    cfg = GlobalConfig.get_instance()
    sc = cfg.server
    sc.model_path = f"preset:{a.model}"
    sc.dtype = "bfloat16"
    sc.tp_size = a.gpus
    sc.max_running_requests = a.batch_size
    sc.max_total_tokens = a.batch_size * (a.input_len + a.output_len) + 4096
    sc.context_length = a.input_len + a.output_len + 64
    br = BenchRunner.create(cfg)
    dev = br.device
    bs, L, out_len = a.batch_size, a.input_len, a.output_len
    tokens_per_step = bs * (L + out_len)

    ids_pinned = make_synthetic_input_ids(batch_size=bs, input_len=L, vocab_size=br.runner.vocab_size, seed=42, pin=True)
    ids_dev = ids_pinned.to(dev)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def one_pass(ids, readback: bool):
        br.clear()
        nxt = br.extend(ids)
        host = [nxt.cpu()] if readback else None
        for _ in range(out_len - 1):
            nxt = br.decode(nxt)
            if readback:
                host.append(nxt.cpu())
        return nxt, host

    for _ in range(max(a.warmup, 3)):
        one_pass(ids_dev, False)
    barrier()

    # ---- device-timed region --------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    graphs = br.runner.cuda_graph_runner
    l0 = ops.launch_count() + (graphs.replayed_kernels if graphs else 0)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * a.steps + 1)]
    pre_ev = []
    barrier()
    ev[0].record()
    for s in range(a.steps):
        br.clear()
        nxt = br.extend(ids_dev)
        ev[2 * s + 1].record()
        for _ in range(out_len - 1):
            nxt = br.decode(nxt)
        ev[2 * s + 2].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[2 * a.steps])
    prefill_ms = [ev[2 * s].elapsed_time(ev[2 * s + 1]) for s in range(a.steps)]
    decode_ms = [ev[2 * s + 1].elapsed_time(ev[2 * s + 2]) for s in range(a.steps)]
    launches = ops.launch_count() + (graphs.replayed_kernels if graphs else 0) - l0
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status(dev.index)

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    total_ms = max_over_ranks(total_ms)
    prefill_med = max_over_ranks(statistics.median(prefill_ms))
    decode_med = max_over_ranks(statistics.median(decode_ms))
    ms_per_step = total_ms / a.steps

    # ---- end-to-end through the public API: pinned host ids in, sampled ids out every step --------
    e2e = None
    if not a.no_e2e:
        one_pass(ids_pinned, True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            one_pass(ids_pinned, True)
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e = {
            "value": tokens_per_step * a.steps / e2e_s, "unit": "tokens/s",
            "h2d_bytes_per_step": int(ids_pinned.numel() * ids_pinned.element_size()),
            "d2h_bytes_per_step": int(out_len * bs * 8),
            "ms_per_step": e2e_s * 1e3 / a.steps,
            "api": "mllm_b200.bench_one_batch.BenchRunner.extend/decode",
        }

    result = {
        "metric": METRIC, "value": tokens_per_step / (ms_per_step / 1e3), "unit": "tokens/s", "n_gpus": a.gpus,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random ids, random-init weights)",
        "impl": "ours",
        "config": {"model": a.model, "global_batch": bs, "seq_len": L, "output_len": out_len,
                   "parallelism": f"tp{a.gpus}", "cuda_graph_decode": graphs is not None,
                   "l2_policy": "inputs larger than L2: every step streams the full weight set (>= 16 GB at TP=1) and the KV pool"},
        "prefill_tokens_per_s": bs * L / (prefill_med / 1e3),
        "decode_tokens_per_s": bs * (out_len - 1) / (decode_med / 1e3),
        "prefill_ms": prefill_med, "decode_ms_per_token": decode_med / (out_len - 1),
        "gpu_launches": int(launches), "clocks": clocks, "e2e": e2e,
    }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result if rank == 0 else {}


# --------------------------------------------------------------------------------------------
# reference arm: unmodified pymllm from baseline/_ref through its own bench_one_batch code
# --------------------------------------------------------------------------------------------
def run_reference(a: argparse.Namespace) -> dict:
    from baseline.reference_arm import run as run_ref

    return run_ref(a, METRIC)


def main() -> None:
    a = parse()
    out = run_reference(a) if a.impl == "reference" else run_ours(a)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()

"""Flagship benchmark: Qwen3-8B-shaped decoder, bf16, one batch of `--batch-size` requests with
input_len 2048 and output_len 128 (prefill + 127 greedy decode steps) — the reference's
``bench_one_batch`` workload — on N GPUs of one node.  With N > 1 the default is tensor parallelism
(``--parallelism tp``): the one batch is sharded over the N GPUs and every layer's partial sums cross
NVLink inside the fused kernels (GEMM with reduce-scatter epilogue, reduce + add + RMSNorm + all-gather,
flag-gated consumer GEMM; the peer-memory reduce in decode) — strong scaling, lower latency per batch.
``--parallelism dp`` runs one full replica of the model per GPU instead, each serving its own batch of
`--batch-size` requests (global batch N x batch, weak scaling, no collective in the timed region).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference --gpus 1 --steps 5 --warmup 3

One *step* is one complete batch: prefill of batch x 2048 seeded random token ids followed by
127 decode steps (128 output tokens per request).  ``value`` is whole-job tokens per second,
``batch * (2048 + 128) / seconds_per_step``, with the step timed on the device by CUDA events
(maximum over ranks).  ``e2e`` repeats the measurement through the public
``BenchRunner.extend`` / ``decode`` API with the prompt ids copied from pinned host memory
and every step's sampled ids read back into pinned host memory (the copy of a step is queued behind
it, the next step is queued, then the host waits for the copy: the host reads every step, one step
behind the launches), timed by the host clock around device synchronisation.  Weights are random-init
(seeded N(0, 0.02)); data are synthetic.
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
    ap.add_argument("--page-size", type=int, default=16, help="slots per KV page of our engine")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--parallelism", choices=["dp", "tp"], default="tp",
                    help="N > 1: tp = one batch sharded over N GPUs (fused NVLink kernels), dp = one replica and one batch per GPU")
    ap.add_argument("--comm-backend", choices=["fused", "nccl"], default="fused",
                    help="tp only: fused = peer-memory kernels of this package, nccl = library all-reduce after o_proj / down_proj")
    ap.add_argument("--device", choices=["cuda", "cpu"], default="cuda",
                    help="cpu runs the same control flow on the host reference ops (flow tests; not a measurement)")
    ap.add_argument("--watchdog-s", type=float, default=1500.0,
                    help="give up (stack dump, error line, exit 3) when the whole run takes longer than this")
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
class _HostEvent:
    """Stand-in for a CUDA event when the flow runs on the host."""

    def __init__(self, enable_timing: bool = True) -> None:
        self.t = 0.0

    def record(self) -> None:
        self.t = time.perf_counter()

    def elapsed_time(self, other: "_HostEvent") -> float:
        return (other.t - self.t) * 1e3

    def synchronize(self) -> None:
        pass


class Watchdog:
    """Bounds the whole run: past the deadline every thread's Python stack goes to stderr, rank 0
    prints a JSON line with an ``error`` field, and the process leaves with status 3 even if a CUDA
    or collective call never returns."""

    def __init__(self, seconds: float, rank: int, gpus: int) -> None:
        self.t0 = time.perf_counter()
        self.phase = "start"
        self.rank = rank
        self.gpus = gpus
        self.done = threading.Event()
        if seconds > 0:
            threading.Thread(target=self._run, args=(seconds,), daemon=True).start()

    def log(self, phase: str) -> None:
        self.phase = phase
        print(f"[bench rank {self.rank} +{time.perf_counter() - self.t0:7.1f}s] {phase}", file=sys.stderr, flush=True)

    def _run(self, seconds: float) -> None:
        if self.done.wait(seconds):
            return
        import faulthandler

        print(f"[bench rank {self.rank}] no result after {seconds:.0f} s, last phase: {self.phase}", file=sys.stderr, flush=True)
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        if self.rank == 0:
            print(json.dumps({"metric": METRIC, "value": None, "n_gpus": self.gpus, "impl": "ours",
                              "error": f"run exceeded {seconds:.0f} s in phase '{self.phase}'"}), flush=True)
        os._exit(3)


def run_ours(a: argparse.Namespace) -> dict:
    import torch
    import torch.distributed as dist

    from mllm_b200 import ops
    from mllm_b200.bench_one_batch import BenchRunner, make_synthetic_input_ids
    from mllm_b200.configs import GlobalConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {a.gpus}")
    wd = Watchdog(a.watchdog_s, rank, a.gpus)
    on_gpu = a.device == "cuda"
    if on_gpu:
        torch.cuda.set_device(local_rank)
    Event = torch.cuda.Event if on_gpu else _HostEvent

    def sync() -> None:
        if on_gpu:
            torch.cuda.synchronize()
    use_tp = world > 1 and a.parallelism == "tp"
    replicas = 1 if (use_tp or world == 1) else world
    if world > 1:
        # host-side group (gloo) for barriers and for reducing the timings; NCCL is brought up
        # only by the tensor-parallel layout, which moves activations between the GPUs
        import datetime

        dist.init_process_group(backend="cpu:gloo,cuda:nccl" if on_gpu else "gloo", timeout=datetime.timedelta(seconds=600))
    wd.log(f"process group ready (world {world}, {'tp' if use_tp else 'dp'})")

    GlobalConfig.reset()
    cfg = GlobalConfig.get_instance()
    sc = cfg.server
    sc.model_path = f"preset:{a.model}"
    sc.dtype = "bfloat16"
    sc.tp_size = a.gpus if use_tp else 1
    if use_tp:
        sc.comm_backend = a.comm_backend
    sc.dp_size = replicas
    sc.max_running_requests = a.batch_size
    sc.max_total_tokens = a.batch_size * (a.input_len + a.output_len + a.page_size) + 4096
    sc.context_length = a.input_len + a.output_len + 64
    # pages of 16 slots: a request's tokens lie in runs of consecutive slots, which the decode-attention kernel
    # fetches as whole boxes from the head-major KV pool
    sc.radix_cache_page_size = a.page_size
    br = BenchRunner.create(cfg, device=None if on_gpu else "cpu")
    wd.log("model runner ready")
    dev = br.device
    bs, L, out_len = a.batch_size, a.input_len, a.output_len
    tokens_per_step = replicas * bs * (L + out_len)   # whole job: every replica serves its own batch

    ids_pinned = make_synthetic_input_ids(batch_size=bs, input_len=L, vocab_size=br.runner.vocab_size,
                                          seed=42 + (rank if replicas > 1 else 0), pin=True)
    ids_dev = ids_pinned.to(dev)

    def reduce_host(v: float, op) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def barrier() -> None:
        sync()
        if world > 1:
            reduce_host(0.0, dist.ReduceOp.SUM)

    # end-to-end passes read every step's token ids back into pinned host memory
    host_ids = torch.empty((out_len, bs), dtype=torch.int64, pin_memory=on_gpu)
    copied = [Event(enable_timing=False), Event(enable_timing=False)]   # step t records copied[t & 1]

    def one_pass(ids, readback: bool):
        """One batch through the public API.  With ``readback`` every step's sampled ids are copied to the host:
        the copy of step t is queued behind step t, step t + 1 is queued next, and only then does the host wait
        for the copy of step t - so the device never idles while the host reads (the ids a step needs are on the
        device already).  Returns the last ids and the host buffer."""
        br.clear()
        nxt = br.extend(ids)
        if not readback:
            for _ in range(out_len - 1):
                nxt = br.decode(nxt)
            return nxt, None
        for t in range(out_len):
            host_ids[t].copy_(nxt.reshape(-1), non_blocking=True)
            copied[t & 1].record()
            if t + 1 < out_len:
                nxt = br.decode(nxt)
            if t > 0:
                copied[(t - 1) & 1].synchronize()      # step t - 1's ids are in host memory now
        copied[(out_len - 1) & 1].synchronize()
        return nxt, host_ids

    for i in range(max(a.warmup, 3)):
        one_pass(ids_dev, False)
        sync()
        wd.log(f"warm-up {i + 1} done")
    barrier()

    # ---- device-timed region --------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0 and on_gpu:
        sampler.start()
    graphs = br.runner.cuda_graph_runner
    l0 = ops.launch_count() + (graphs.replayed_kernels if graphs else 0)
    ev = [Event(enable_timing=True) for _ in range(2 * a.steps + 1)]
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
    sync()
    clocks = sampler.stop() if rank == 0 and on_gpu else None
    if on_gpu:
        ops.check_status(dev.index)
    wd.log("timed region done")

    MAX, SUM = (dist.ReduceOp.MAX, dist.ReduceOp.SUM) if world > 1 else (None, None)
    total_ms = reduce_host(total_ms, MAX)
    prefill_med = reduce_host(statistics.median(prefill_ms), MAX)
    decode_med = reduce_host(statistics.median(decode_ms), MAX)
    launches_all = int(reduce_host(float(launches), SUM))
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
        e2e_s = reduce_host(time.perf_counter() - t0, MAX)
        e2e = {
            "value": tokens_per_step * a.steps / e2e_s, "unit": "tokens/s",
            "h2d_bytes_per_step": int(replicas * ids_pinned.numel() * ids_pinned.element_size()),
            "d2h_bytes_per_step": int(replicas * out_len * bs * 8),
            "ms_per_step": e2e_s * 1e3 / a.steps,
            "api": "mllm_b200.bench_one_batch.BenchRunner.extend/decode",
            "readback": "each step's ids to pinned host memory, awaited after the next step is queued",
        }
        wd.log("end-to-end region done")

    layout = f"tp{a.gpus}" if use_tp else f"dp{a.gpus}"
    comm_info = None
    if use_tp:
        from mllm_b200.parallel.symm import get_tp_comm

        comm = get_tp_comm()
        comm_info = {"path": "fused peer-memory kernels" if comm is not None else "nccl all-reduce",
                     "fused_prefill_calls": int(comm.epoch) if comm is not None else 0,
                     "prefill_rows_cap": int(comm.prefill.rows_cap) if comm is not None and comm.prefill is not None else 0}
    result = {
        "metric": METRIC, "value": tokens_per_step / (ms_per_step / 1e3), "unit": "tokens/s", "n_gpus": a.gpus,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if use_tp else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded random ids, random-init weights)",
        "impl": "ours", **({} if on_gpu else {"device": "cpu", "note": "host flow run: not a measurement"}),
        "config": {"model": a.model, "global_batch": replicas * bs, "per_gpu_batch": bs if not use_tp else None,
                   "seq_len": L, "output_len": out_len,
                   "parallelism": layout, "cuda_graph_decode": graphs is not None, "kv_page_size": a.page_size,
                   "l2_policy": "inputs larger than L2: every step streams the full weight set (>= 16 GB per replica) and the KV pool"},
        "prefill_tokens_per_s": replicas * bs * L / (prefill_med / 1e3),
        "decode_tokens_per_s": replicas * bs * (out_len - 1) / (decode_med / 1e3),
        "prefill_ms": prefill_med, "decode_ms_per_token": decode_med / (out_len - 1),
        # the batch's time to first token and time per output token, median over the timed steps (max over ranks)
        "p50_ttft_ms": prefill_med, "p50_tpot_ms": decode_med / (out_len - 1),
        "gpu_launches": launches_all, "gpu_launches_per_rank": int(launches), "clocks": clocks, "e2e": e2e,
        "comm": comm_info,
    }
    if world > 1:
        barrier()
        dist.destroy_process_group()
    wd.done.set()
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

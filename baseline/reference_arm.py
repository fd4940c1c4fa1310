"""Reference arm of bench.py: the unmodified pymllm (installed under ``baseline/_ref``) driven
through its own ``bench_one_batch`` code path — ``parse_args`` -> ``PymllmBenchRunner.create`` ->
``run_single_setting`` — on the same workload as our arm.  Nothing of mllm_b200's models,
kernels or engine is on that path; mllm_b200 only writes the seeded random-init checkpoint
directory the reference loads (it can only load weights from files).
"""

from __future__ import annotations

import json
import os
import statistics
import sys
import traceback
from pathlib import Path

REF_ROOT = Path(__file__).resolve().parent / "_ref"


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}


class _Ranks:
    """Lock-step helper for N independent reference replicas (one per GPU): after every phase the ranks
    exchange an error string, so a failure on one rank ends all of them together instead of leaving the
    others waiting.  The exchange goes through the launcher's key-value store only; no process group is
    created, so inside each replica ``torch.distributed`` looks exactly as it does in a single-GPU run."""

    def __init__(self) -> None:
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.store = None
        self.round = 0
        if self.world > 1:
            import datetime

            from torch.distributed.rendezvous import rendezvous

            self.store, _, _ = next(rendezvous("env://", timeout=datetime.timedelta(seconds=1200)))

    def gather(self, obj):
        if self.world == 1:
            return [obj]
        import pickle

        self.round += 1
        self.store.set(f"mllm_b200_ref/{self.round}/{self.rank}", pickle.dumps(obj))
        return [pickle.loads(self.store.get(f"mllm_b200_ref/{self.round}/{r}")) for r in range(self.world)]

    def check(self, phase: str, err=None) -> None:
        errs = [e for e in self.gather(err) if e]
        if errs:
            raise RuntimeError(f"{phase}: {errs[0]}")

    def phase(self, name: str, fn, only_rank0: bool = False):
        out, err = None, None
        if not only_rank0 or self.rank == 0:
            try:
                out = fn()
            except BaseException as exc:  # noqa: BLE001
                traceback.print_exc(file=sys.stderr)
                err = f"rank {self.rank}: {type(exc).__name__}: {exc}"
        self.check(name, err)
        return out


def run(a, metric: str) -> dict:
    """N > 1: pymllm has no tensor-parallel runtime (its ServerConfig has no tp_size, the process group is
    never initialised outside a unit test, the models use non-parallel linears), so the reference scales
    the way our default arm does: one unmodified replica per GPU, each serving its own batch."""
    ranks = _Ranks()
    if ranks.world != a.gpus:
        return _unavailable(f"--gpus {a.gpus} but WORLD_SIZE={ranks.world}") if ranks.rank == 0 else {}
    if not (REF_ROOT / "pymllm").exists():
        return _unavailable("baseline/_ref/pymllm not installed") if ranks.rank == 0 else {}
    try:
        out = _run(a, metric, ranks)
    except BaseException as exc:  # noqa: BLE001 - the driver needs a JSON line, not a traceback
        traceback.print_exc(file=sys.stderr)
        out = _unavailable(f"reference failed on this box: {type(exc).__name__}: {exc}")
    return out if ranks.rank == 0 else {}


def _run(a, metric: str, ranks: "_Ranks") -> dict:
    import torch

    sys.path.insert(0, str(REF_ROOT))
    from mllm_b200.io.random_checkpoint import write_random_checkpoint

    torch.cuda.set_device(ranks.local)
    ckpt_dir = f"/tmp/mllm_b200_ref_ckpt/{a.model}"
    ranks.phase("checkpoint", lambda: write_random_checkpoint(a.model, ckpt_dir, seed=0), only_rank0=True)
    ckpt = Path(ckpt_dir)
    torch.cuda.empty_cache()

    from pymllm import bench_one_batch as rb

    argv = [
        "--server.model_path", str(ckpt), "--server.dtype", "bfloat16",
        "--batch-size", str(a.batch_size), "--input-len", str(a.input_len), "--output-len", str(a.output_len),
        "--result-filename", f"/tmp/mllm_b200_ref_bench_{ranks.rank}.jsonl",
        "--server.base_gpu_id", str(ranks.local),
    ]

    def build():
        cfg, args = rb.parse_args(argv)
        rb._load_hf_config(cfg)
        rb._align_runner_capacity_with_batch_sizes(cfg, args.batch_size)
        return args, rb.PymllmBenchRunner.create(cfg)

    args, runner = ranks.phase("load", build)
    setting = rb.generate_settings(args)[0]
    tokens = ranks.world * setting.batch_size * (setting.input_len + setting.output_len)

    def one(record: bool):
        return rb.run_single_setting(bench_runner=runner, args=args, setting=setting, seed=args.seed,
                                     record_result=record, allow_profile=False)

    warm = max(a.warmup, 3)

    def warm_up():
        for _ in range(warm):
            one(False)
        torch.cuda.synchronize()

    ranks.phase("warm-up", warm_up)          # also the barrier in front of the timed region
    rows = []

    def timed():
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(a.steps):
            rows.append(one(True))
        ev1.record()
        torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) / a.steps

    mine = ranks.phase("timed region", timed)
    ms_per_step = max(ranks.gather(mine))    # the job is as slow as its slowest replica
    rows = [r for r in rows if r]
    value = tokens / (ms_per_step / 1e3)
    out = {
        "impl": "reference", "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": ranks.world, "steps": a.steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random ids, random-init weights)",
        "config": {"model": a.model, "global_batch": ranks.world * setting.batch_size, "per_gpu_batch": setting.batch_size,
                   "seq_len": setting.input_len, "output_len": setting.output_len, "parallelism": f"dp{ranks.world}",
                   "path": "pymllm.bench_one_batch.run_single_setting (stock)"},
        "e2e": {"value": value, "unit": "tokens/s", "note": "the reference's bench loop is already end to end: "
                "ids are generated on the host and copied in, each step is synchronised"},
    }
    if rows:
        out["prefill_tokens_per_s"] = statistics.median(r["prefill_throughput"] for r in rows)
        out["decode_tokens_per_s"] = statistics.median(r["median_decode_throughput"] for r in rows)
        out["reference_reported_overall_throughput"] = statistics.median(r["overall_throughput"] for r in rows)
        if all("prefill_latency" in r for r in rows):
            out["p50_ttft_ms"] = statistics.median(r["prefill_latency"] for r in rows) * 1e3
        if all("median_decode_latency" in r for r in rows):
            out["p50_tpot_ms"] = statistics.median(r["median_decode_latency"] for r in rows) * 1e3
    runner.shutdown()
    return out

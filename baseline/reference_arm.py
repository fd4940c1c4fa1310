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


def run(a, metric: str) -> dict:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if a.gpus > 1 or world > 1:
        # pymllm has no tensor-parallel runtime: ServerConfig has no tp_size, the process group is
        # never initialised outside a unit test and the models use non-parallel linears.
        return _unavailable("reference pymllm is single-GPU only (no tp_size, parallel_state never initialised)") \
            if rank == 0 else {}
    if not (REF_ROOT / "pymllm").exists():
        return _unavailable("baseline/_ref/pymllm not installed")
    try:
        return _run(a, metric)
    except BaseException as exc:  # noqa: BLE001 - the driver needs a JSON line, not a traceback
        traceback.print_exc(file=sys.stderr)
        return _unavailable(f"reference failed on this box: {type(exc).__name__}: {exc}")


def _run(a, metric: str) -> dict:
    import torch

    sys.path.insert(0, str(REF_ROOT))
    from mllm_b200.io.random_checkpoint import write_random_checkpoint

    ckpt = write_random_checkpoint(a.model, f"/tmp/mllm_b200_ref_ckpt/{a.model}", seed=0)
    torch.cuda.empty_cache()

    from pymllm import bench_one_batch as rb

    argv = [
        "--server.model_path", str(ckpt), "--server.dtype", "bfloat16",
        "--batch-size", str(a.batch_size), "--input-len", str(a.input_len), "--output-len", str(a.output_len),
        "--result-filename", "/tmp/mllm_b200_ref_bench.jsonl",
    ]
    cfg, args = rb.parse_args(argv)
    rb._load_hf_config(cfg)
    rb._align_runner_capacity_with_batch_sizes(cfg, args.batch_size)
    runner = rb.PymllmBenchRunner.create(cfg)
    setting = rb.generate_settings(args)[0]
    tokens = setting.batch_size * (setting.input_len + setting.output_len)

    def one(record: bool):
        return rb.run_single_setting(bench_runner=runner, args=args, setting=setting, seed=args.seed,
                                     record_result=record, allow_profile=False)

    warm = max(a.warmup, 3)
    for _ in range(warm):
        one(False)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rows = []
    ev0.record()
    for _ in range(a.steps):
        rows.append(one(True))
    ev1.record()
    torch.cuda.synchronize()
    ms_per_step = ev0.elapsed_time(ev1) / a.steps
    rows = [r for r in rows if r]
    value = tokens / (ms_per_step / 1e3)
    out = {
        "impl": "reference", "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random ids, random-init weights)",
        "config": {"model": a.model, "global_batch": setting.batch_size, "seq_len": setting.input_len,
                   "output_len": setting.output_len, "parallelism": "tp1",
                   "path": "pymllm.bench_one_batch.run_single_setting (stock)"},
        "e2e": {"value": value, "unit": "tokens/s", "note": "the reference's bench loop is already end to end: "
                "ids are generated on the host and copied in, each step is synchronised"},
    }
    if rows:
        out["prefill_tokens_per_s"] = statistics.median(r["prefill_throughput"] for r in rows)
        out["decode_tokens_per_s"] = statistics.median(r["median_decode_throughput"] for r in rows)
        out["reference_reported_overall_throughput"] = statistics.median(r["overall_throughput"] for r in rows)
    runner.shutdown()
    return out

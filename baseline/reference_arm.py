"""Reference arm of bench.py: the unmodified pymllm (installed under ``baseline/_ref``) driven
through its own ``bench_one_batch`` code path — ``parse_args`` -> ``PymllmBenchRunner.create`` ->
``run_single_setting`` — on the same workload as our arm.  Nothing of mllm_b200's models,
kernels or engine is on that path; mllm_b200 only writes the seeded random-init checkpoint
directory the reference loads (it can only load weights from files).

N > 1, tensor-parallel layout (``--parallelism tp``, the default): pymllm ships the parallel building
blocks (``ColumnParallelLinear`` / ``RowParallelLinear`` with an NCCL all-reduce,
``parallel_state.initialize_model_parallel``) but no runtime that uses them, so this arm assembles the
tensor-parallel Qwen3 from the reference's own files, with these substitutions, all made by binding
names of the reference's modules before its model is built (no reference file is edited):

* every rank builds the reference's ``Qwen3ForCausalLM`` from a ``config.json`` that names this rank's
  share of the heads and of the MLP width — its fused ``qkv_proj`` / ``gate_up_proj`` are then exactly the
  column-parallel shards;
* the two projections that close a block, ``o_proj`` and ``down_proj``, which the reference's Qwen3 builds as
  plain ``Linear``, are built as the reference's ``RowParallelLinear`` (all-reduce over its NCCL group after the
  GEMM; pymllm/layers/linear.py:246-268);
* embedding and lm_head stay replicated, as the reference's Qwen3 has them (no vocabulary-parallel head);
* the process group is NCCL, brought up by ``torch.distributed`` and handed to the reference's
  ``initialize_model_parallel``; the reference's CUDA-graph runner captures the all-reduces with the rest of
  the decode step.

``--parallelism dp`` keeps one unmodified replica per GPU.
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
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and getattr(a, "parallelism", "tp") == "tp":
        return run_tp(a, metric)
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
        "config": _config(a, setting.batch_size, ranks.world, f"dp{ranks.world}"),
        "path": "pymllm.bench_one_batch.run_single_setting (stock)",
        "e2e": {"value": value, "unit": "tokens/s",
                "h2d_bytes_per_step": ranks.world * setting.batch_size * setting.input_len * 4,
                "d2h_bytes_per_step": ranks.world * setting.output_len * setting.batch_size * 8,
                "note": "the reference's bench loop is already end to end: ids are generated on the host and "
                        "copied in, each step is synchronised and its ids read"},
    }
    _add_row_stats(out, rows)
    runner.shutdown()
    return out


# --------------------------------------------------------------------------------------------
# tensor-parallel reference: the reference's own parallel layers under its own bench loop
# --------------------------------------------------------------------------------------------
def run_tp(a, metric: str) -> dict:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != a.gpus:
        return _unavailable(f"--gpus {a.gpus} but WORLD_SIZE={world}") if rank == 0 else {}
    if not (REF_ROOT / "pymllm").exists():
        return _unavailable("baseline/_ref/pymllm not installed") if rank == 0 else {}
    try:
        out = _run_tp(a, metric, world, rank)
    except BaseException as exc:  # noqa: BLE001 - the driver needs a JSON line, not a traceback
        traceback.print_exc(file=sys.stderr)
        out = _unavailable(f"tensor-parallel reference failed on this box: {type(exc).__name__}: {exc}")
        if rank == 0:
            print(json.dumps(out), flush=True)
        os._exit(0)      # a rank that failed alone must not leave the others waiting in a collective
    return out if rank == 0 else {}


def _run_tp(a, metric: str, world: int, rank: int) -> dict:
    import datetime

    import torch
    import torch.distributed as dist

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl", timeout=datetime.timedelta(seconds=600),
                            device_id=torch.device("cuda", local))
    sys.path.insert(0, str(REF_ROOT))
    from mllm_b200.io.random_checkpoint import write_random_checkpoint

    # one directory for all ranks: the shard's weights are random anyway, o_proj / down_proj are full width
    # and every rank's row-parallel loader cuts out its own slice
    ckpt_dir = f"/tmp/mllm_b200_ref_ckpt/{a.model}-tp{world}"
    err = None
    if rank == 0:
        try:
            write_random_checkpoint(a.model, ckpt_dir, seed=0, tp_shard=world)
        except BaseException as exc:  # noqa: BLE001
            err = f"{type(exc).__name__}: {exc}"
    box = [err]
    dist.broadcast_object_list(box, src=0)
    if box[0]:
        raise RuntimeError(f"checkpoint: {box[0]}")
    torch.cuda.empty_cache()

    from pymllm.orchestrator import parallel_state as ref_ps

    ref_ps.initialize_model_parallel(tensor_model_parallel_size=world, backend="nccl")
    import pymllm.layers.mlp as ref_mlp
    import pymllm.models.qwen3 as ref_qwen3
    from pymllm.layers.linear import RowParallelLinear

    def row_parallel(in_features, out_features, bias=False, quant_method=None):
        # the model asks for this rank's input width; the reference's layer takes the width before the split
        return RowParallelLinear(in_features * world, out_features, bias=bias, reduce_output=True,
                                 quant_method=quant_method)

    ref_qwen3.Linear = row_parallel        # o_proj (the only Linear Qwen3Attention builds with fused qkv)
    ref_mlp.Linear = row_parallel          # down_proj (the only Linear MLP builds with fused gate_up)

    from pymllm import bench_one_batch as rb

    argv = [
        "--server.model_path", ckpt_dir, "--server.dtype", "bfloat16",
        "--batch-size", str(a.batch_size), "--input-len", str(a.input_len), "--output-len", str(a.output_len),
        "--result-filename", f"/tmp/mllm_b200_ref_bench_tp_{rank}.jsonl",
        "--server.base_gpu_id", str(local),
    ]
    cfg, args = rb.parse_args(argv)
    rb._load_hf_config(cfg)
    rb._align_runner_capacity_with_batch_sizes(cfg, args.batch_size)
    runner = rb.PymllmBenchRunner.create(cfg)
    n_row = sum(isinstance(m, RowParallelLinear) for m in runner.model_runner.model.modules()) \
        if hasattr(runner, "model_runner") else -1
    setting = rb.generate_settings(args)[0]
    tokens = setting.batch_size * (setting.input_len + setting.output_len)

    def one(record: bool):
        return rb.run_single_setting(bench_runner=runner, args=args, setting=setting, seed=args.seed,
                                     record_result=record, allow_profile=False)

    def host_max(v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warm = max(a.warmup, 3)
    for _ in range(warm):
        one(False)
    torch.cuda.synchronize()
    host_max(0.0)
    rows = []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(a.steps):
        rows.append(one(True))
    ev1.record()
    torch.cuda.synchronize()
    ms_per_step = host_max(ev0.elapsed_time(ev1) / a.steps)
    rows = [r for r in rows if r]
    value = tokens / (ms_per_step / 1e3)
    ids_bytes = setting.batch_size * setting.input_len * 4
    out = {
        "impl": "reference", "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random ids, random-init weights)",
        "config": _config(a, setting.batch_size, None, f"tp{world}"),
        "path": "pymllm.bench_one_batch.run_single_setting over the reference's Qwen3 with its RowParallelLinear "
                "(NCCL all-reduce) closing every block; embedding and lm_head replicated",
        "row_parallel_layers": n_row,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": ids_bytes,
                "d2h_bytes_per_step": setting.output_len * setting.batch_size * 8,
                "note": "the reference's bench loop is already end to end: ids are generated on the host and copied "
                        "in, each step is synchronised and its ids read"},
    }
    _add_row_stats(out, rows)
    dist.barrier()
    runner.shutdown()
    dist.destroy_process_group()
    return out


def _config(a, per_gpu_batch, replicas, layout: str) -> dict:
    """The same keys, in the same order, as our arm's ``config``."""
    return {"model": a.model, "global_batch": per_gpu_batch * (replicas or 1),
            "per_gpu_batch": per_gpu_batch if replicas else None, "seq_len": a.input_len, "output_len": a.output_len,
            "parallelism": layout, "cuda_graph_decode": True, "kv_page_size": 1,
            "l2_policy": "inputs larger than L2: every step streams the full weight set (>= 16 GB per replica) and the KV pool"}


def _add_row_stats(out: dict, rows) -> None:
    if not rows:
        return
    out["prefill_tokens_per_s"] = statistics.median(r["prefill_throughput"] for r in rows)
    out["decode_tokens_per_s"] = statistics.median(r["median_decode_throughput"] for r in rows)
    out["reference_reported_overall_throughput"] = statistics.median(r["overall_throughput"] for r in rows)
    if all("prefill_latency" in r for r in rows):
        out["p50_ttft_ms"] = statistics.median(r["prefill_latency"] for r in rows) * 1e3
    if all("median_decode_latency" in r for r in rows):
        out["p50_tpot_ms"] = statistics.median(r["median_decode_latency"] for r in rows) * 1e3

"""One-batch latency benchmark that drives :class:`ModelRunner` directly (no scheduler).

Command line, sweep semantics, timing method and JSONL schema follow
pymllm/bench_one_batch.py:111-218,312-353,943-1121: for every
``batch x input_len x output_len`` one static prefill and ``output_len - 1`` decode steps are
timed between ``torch.cuda.synchronize()`` calls; rows carry ``prefill_latency``,
``prefill_throughput``, ``median_decode_latency``, ``median_decode_throughput``,
``total_latency`` and ``overall_throughput``; a short warm-up run comes first; a setting that
does not fit the KV pool is skipped; ``max_running_requests`` is raised to the largest batch
so CUDA graphs cover it.  Additions: every row also carries device-side (CUDA event) timings,
``--server.tp_size`` runs under ``torchrun`` report the max over ranks, and ``preset:<name>``
model paths run random-init weights without a checkpoint directory.

    python -m mllm_b200.bench_one_batch --server.model_path preset:qwen3-8b \
        --batch-size 1 8 --input-len 2048 --output-len 128
"""

from __future__ import annotations

import argparse
import json
import logging
import statistics
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

import torch

from .configs import GlobalConfig, make_args, read_args
from .executor import ModelRunner, load_hf_config
from .parallel import state as pstate

logger = logging.getLogger("mllm_b200.bench_one_batch")


@dataclass
class BenchArgs:
    run_name: str = "default"
    batch_size: List[int] = field(default_factory=lambda: [1])
    input_len: List[int] = field(default_factory=lambda: [256, 512, 1024])
    output_len: List[int] = field(default_factory=lambda: [128])
    result_filename: Path = Path("mllm_b200_bench_one_batch.jsonl")
    log_decode_step: int = 0
    seed: int = 42
    profile: bool = False
    profile_record_shapes: bool = False
    profile_activities: List[str] = field(default_factory=lambda: ["CPU", "GPU"])
    profile_stage: str = "all"
    profile_filename_prefix: str = "mllm_b200_bench_one_batch"
    profile_start_step: Optional[int] = None
    profile_steps: int = 1
    skip_warmup: bool = False
    image_path: Optional[Path] = None
    synthetic_image: bool = False
    prompt: str = "Describe this image."
    input_len_was_provided: bool = False
    correctness_test: bool = False


@dataclass(frozen=True)
class BenchSetting:
    batch_size: int
    input_len: int
    output_len: int


def _positive_int(v: str) -> int:
    i = int(v)
    if i <= 0:
        raise argparse.ArgumentTypeError(f"Expected a positive integer, got {v!r}")
    return i


def _non_negative_int(v: str) -> int:
    i = int(v)
    if i < 0:
        raise argparse.ArgumentTypeError(f"Expected a non-negative integer, got {v!r}")
    return i


def add_bench_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    g = parser.add_argument_group("bench_one_batch", "Options of the one-batch benchmark.")
    g.add_argument("--run-name", default=BenchArgs.run_name)
    g.add_argument("--batch-size", nargs="+", type=_positive_int, default=[1])
    g.add_argument("--input-len", nargs="+", type=_positive_int, default=[256, 512, 1024])
    g.add_argument("--output-len", nargs="+", type=_positive_int, default=[128])
    g.add_argument("--result-filename", type=Path, default=BenchArgs.result_filename)
    g.add_argument("--log-decode-step", type=_non_negative_int, default=0)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--profile", action="store_true")
    g.add_argument("--profile-record-shapes", action="store_true")
    g.add_argument("--profile-activities", nargs="+", choices=["CPU", "GPU", "CUDA_PROFILER"], default=["CPU", "GPU"])
    g.add_argument("--profile-stage", choices=["all", "prefill", "decode"], default="all")
    g.add_argument("--profile-filename-prefix", default=BenchArgs.profile_filename_prefix)
    g.add_argument("--profile-start-step", type=_non_negative_int, default=None)
    g.add_argument("--profile-steps", type=_positive_int, default=1)
    g.add_argument("--skip-warmup", action="store_true")
    g.add_argument("--image", "--image-path", dest="image_path", type=Path, default=None)
    g.add_argument("--synthetic-image", action="store_true",
                   help="multimodal run with a seeded uniform-random 448x448 image per request")
    g.add_argument("--prompt", default=BenchArgs.prompt)
    g.add_argument("--correct", "--correctness-test", dest="correctness_test", action="store_true")
    return parser


def make_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="python -m mllm_b200.bench_one_batch",
                                     description="Direct ModelRunner one-batch benchmark.")
    make_args(parser)
    add_bench_args(parser)
    return parser


def parse_args(argv: Optional[Sequence[str]] = None):
    parser = make_parser()
    cli = list(sys.argv[1:] if argv is None else argv)
    cfg = read_args(argv=cli, parser=parser)
    ns = parser.parse_args(cli)
    given = any(a == "--input-len" or a.startswith("--input-len=") for a in cli)
    args = BenchArgs(
        run_name=ns.run_name, batch_size=list(ns.batch_size), input_len=list(ns.input_len),
        output_len=list(ns.output_len), result_filename=Path(ns.result_filename),
        log_decode_step=ns.log_decode_step, seed=ns.seed, profile=ns.profile,
        profile_record_shapes=ns.profile_record_shapes, profile_activities=list(ns.profile_activities),
        profile_stage=ns.profile_stage, profile_filename_prefix=ns.profile_filename_prefix,
        profile_start_step=ns.profile_start_step, profile_steps=ns.profile_steps, skip_warmup=ns.skip_warmup,
        image_path=ns.image_path, synthetic_image=ns.synthetic_image, prompt=ns.prompt, input_len_was_provided=given,
        correctness_test=ns.correctness_test,
    )
    return cfg, args


def generate_settings(args: BenchArgs) -> List[BenchSetting]:
    input_lens = [0] if args.image_path is not None and not args.input_len_was_provided else args.input_len
    return [BenchSetting(b, i, o) for b in args.batch_size for i in input_lens for o in args.output_len]


def make_synthetic_input_ids(*, batch_size: int, input_len: int, vocab_size: int, seed: int,
                             device="cpu", pin: bool = False) -> torch.Tensor:
    """Seeded uniform ids in ``[0, min(vocab, 10000))`` generated on the host."""
    upper = max(1, min(int(vocab_size or 10000), 10000))
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    ids = torch.randint(0, upper, (batch_size, input_len), generator=g, dtype=torch.int32, device="cpu")
    if pin and torch.cuda.is_available():
        ids = ids.pin_memory()
    return ids if str(device) == "cpu" else ids.to(device)


def make_multimodal_inputs(*, hf_config, batch_size: int, input_len: int, image: Optional[torch.Tensor], seed: int):
    """One image per request followed/preceded by seeded text ids so that every request has ``input_len``
    tokens (``input_len == 0``: just the image block and a short text tail).  ``image`` is uint8 [H, W, 3];
    None makes a seeded uniform-random 448 x 448 one.  Returns ``(ids [B, L], pixel_values, grid_thw)``."""
    from .utils.image_processor import image_token_count, preprocess_image

    vc = hf_config.vision_config
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    if image is None:
        image = torch.randint(0, 256, (448, 448, 3), generator=g, dtype=torch.uint8)
    merge = getattr(vc, "spatial_merge_size", 2)
    pix, grid = preprocess_image(image, vc.patch_size, merge, getattr(vc, "temporal_patch_size", 2))
    n_img = image_token_count(grid, merge)
    block = [hf_config.vision_start_token_id] + [hf_config.image_token_id] * n_img + [hf_config.vision_end_token_id]
    L = max(input_len, len(block) + 8)
    tc = getattr(hf_config, "text_config", hf_config)
    special = {hf_config.image_token_id, hf_config.vision_start_token_id, hf_config.vision_end_token_id,
               getattr(hf_config, "video_token_id", -1)}
    upper = max(2, min(int(tc.vocab_size), 10000))
    rows = []
    for _ in range(batch_size):
        text = torch.randint(0, upper, (L - len(block),), generator=g, dtype=torch.int64).tolist()
        text = [t if t not in special else 0 for t in text]
        head = min(4, len(text))
        rows.append(text[:head] + block + text[head:])
    ids = torch.tensor(rows, dtype=torch.int32)
    return ids, pix.repeat(batch_size, 1), grid.repeat(batch_size, 1)


def load_image(path) -> torch.Tensor:
    """uint8 [H, W, 3] from an image file (PIL if present) or a ``.npy`` / ``.pt`` array."""
    p = str(path)
    if p.endswith(".npy"):
        import numpy as np

        return torch.from_numpy(np.load(p)).to(torch.uint8)
    if p.endswith(".pt"):
        return torch.load(p).to(torch.uint8)
    from PIL import Image
    import numpy as np

    return torch.from_numpy(np.asarray(Image.open(p).convert("RGB"))).to(torch.uint8)


def _safe_div(a: float, b: float) -> float:
    return float(a) / float(b) if b else 0.0


def summarize_latencies(*, setting: BenchSetting, prefill_latency: float, decode_latencies: Sequence[float],
                        run_name: str, device: str, dtype: str, cuda_graph: bool,
                        extra: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    med = float(statistics.median(decode_latencies)) if decode_latencies else 0.0
    total = float(prefill_latency + sum(decode_latencies))
    row = {
        "run_name": run_name, "batch_size": setting.batch_size, "input_len": setting.input_len,
        "output_len": setting.output_len, "prefill_latency": float(prefill_latency),
        "prefill_throughput": _safe_div(setting.batch_size * setting.input_len, prefill_latency),
        "median_decode_latency": med, "median_decode_throughput": _safe_div(setting.batch_size, med),
        "total_latency": total,
        "overall_throughput": _safe_div(setting.batch_size * (setting.input_len + setting.output_len), total),
        "device": device, "dtype": dtype, "cuda_graph": cuda_graph,
    }
    if extra:
        row.update(extra)
    return row


class BenchRunner:
    """Minimal request bookkeeping around a ModelRunner: one static batch, prefill then decode."""

    def __init__(self, runner: ModelRunner) -> None:
        self.runner = runner
        self.device = runner.device
        self.slots: List[int] = []
        self.seq_len = 0
        self.batch = 0
        self._slots_dev: Optional[torch.Tensor] = None
        self._seq_lens: Optional[torch.Tensor] = None

    @classmethod
    def create(cls, cfg: GlobalConfig, hf_config=None, device: Optional[str] = None) -> "BenchRunner":
        sc = cfg.server
        if sc.world_size > 1:
            pstate.init_distributed()
            if not pstate.model_parallel_is_initialized():
                pstate.initialize_model_parallel(tp_size=sc.tp_size, ep_size=sc.ep_size, pp_size=sc.pp_size)
        import os

        gpu = sc.base_gpu_id + int(os.environ.get("LOCAL_RANK", "0"))
        runner = ModelRunner(sc, hf_config=hf_config, gpu_id=gpu, quantization_method=cfg.quantization.method,
                             kv_cache_dtype=cfg.quantization.kv_cache_dtype, device=device)
        runner.initialize()
        return cls(runner)

    def clear(self) -> None:
        r = self.runner
        r.req_to_token_pool.clear()
        r.token_to_kv_pool_allocator.clear()
        self.slots, self.seq_len, self.batch = [], 0, 0
        self._own, self._used = None, 0

    def max_batch_size_for(self, input_len: int, output_len: int) -> int:
        return self.runner.max_total_num_tokens // max(1, input_len + output_len)

    @torch.no_grad()
    def extend(self, input_ids: torch.Tensor, **extra) -> torch.Tensor:
        """``input_ids`` [B, L] (host or device). Returns the first generated token per request."""
        r = self.runner
        bs, L = input_ids.shape
        slots = r.req_to_token_pool.alloc(bs)
        # every request owns whole pages: its prompt starts a run of consecutive slots and what is left of its
        # last page serves its first decode steps (with page size 1 this is one plain allocation)
        page = getattr(r.token_to_kv_pool_allocator, "page_size", 1)
        per_req = -(-L // page) * page
        got = r.token_to_kv_pool_allocator.alloc(bs * per_req)
        if slots is None or got is None:
            raise RuntimeError("bench batch does not fit the KV pool")
        self._own = got.view(bs, per_req)
        self._used = L
        loc = self._own[:, :L].reshape(-1)
        self.slots, self.batch, self.seq_len = slots, bs, L
        self._slots_dev = torch.tensor(slots, dtype=torch.int32).to(self.device, non_blocking=True)
        r.req_to_token_pool.req_to_token[self._slots_dev.long(), :L] = loc.view(bs, L).to(torch.int32)
        ids = input_ids.to(self.device, non_blocking=True).reshape(-1).to(torch.int64)
        lens = torch.full((bs,), L, dtype=torch.int32, device=self.device)
        self._seq_lens = lens.clone()
        fb = r.prepare_forward_batch_extend(
            ids, self._slots_dev, lens, lens, torch.zeros_like(lens), loc,
            extend_seq_lens_cpu=[L] * bs, extend_prefix_lens_cpu=[0] * bs, **extra)
        out = r.forward(fb)
        self._mrope_deltas = fb.mrope_position_deltas
        self.last_forward_batch = fb
        return r.sample(out)

    @torch.no_grad()
    def decode(self, last_ids: torch.Tensor) -> torch.Tensor:
        r = self.runner
        bs = self.batch
        page = getattr(r.token_to_kv_pool_allocator, "page_size", 1)
        if self._used == self._own.shape[1]:       # every request's last page is full: one more page each
            more = r.token_to_kv_pool_allocator.alloc(bs * page)
            if more is None:
                raise RuntimeError("KV pool exhausted during decode")
            self._own = torch.cat([self._own, more.view(bs, page)], dim=1)
        graphs = r.cuda_graph_runner
        if (graphs is not None and self.device.type == "cuda" and not getattr(r.model, "uses_mrope", False)
                and graphs.captured_size_for(bs) == bs and last_ids.is_cuda and last_ids.dtype == torch.int64):
            # one kernel does the step's bookkeeping (slot, request table, lengths, positions) and writes the
            # inputs where the captured graph reads them; then the graph is replayed
            from . import ops

            ops.ext().decode_prepare(last_ids.contiguous(), self._slots_dev, self._own, self._used, self._seq_lens,
                                     r.req_to_token_pool.req_to_token, graphs.input_ids, graphs.req_pool_indices,
                                     graphs.seq_lens, graphs.out_cache_loc, graphs.positions)
            self._used += 1
            self.seq_len += 1
            return graphs.replay_static(bs).next_token_ids
        loc = self._own[:, self._used].contiguous()
        self._used += 1
        r.req_to_token_pool.req_to_token[self._slots_dev.long(), self.seq_len] = loc.to(torch.int32)
        self.seq_len += 1
        self._seq_lens += 1
        extra = {}
        if getattr(r.model, "uses_mrope", False):
            pos = (self._seq_lens - 1).to(torch.int64)
            if getattr(self, "_mrope_deltas", None) is not None:
                pos = pos + self._mrope_deltas
            extra["mrope_positions"] = pos.unsqueeze(0).expand(3, -1).contiguous()
        fb = r.prepare_forward_batch_decode(last_ids.to(self.device, non_blocking=True).to(torch.int64),
                                            self._slots_dev, self._seq_lens, loc, max_seq_len=self.seq_len, **extra)
        out = r.forward(fb)
        ids = getattr(out, "next_token_ids", None)
        return ids if ids is not None else r.sample(out)


def _sync(device) -> None:
    if torch.device(device).type == "cuda":
        torch.cuda.synchronize(device)


def _timed_call(device, fn):
    _sync(device)
    t0 = time.perf_counter()
    out = fn()
    _sync(device)
    return time.perf_counter() - t0, out


def _max_over_ranks(value: float, device) -> float:
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_single_setting(*, bench_runner: BenchRunner, args: BenchArgs, setting: BenchSetting, seed: int,
                       record_result: bool) -> Optional[Dict[str, Any]]:
    br = bench_runner
    br.clear()
    dev = br.device
    if setting.batch_size > br.max_batch_size_for(setting.input_len, setting.output_len):
        logger.info("skipping (batch_size=%d, input_len=%d, output_len=%d): exceeds KV capacity %d tokens",
                    setting.batch_size, setting.input_len, setting.output_len, br.runner.max_total_num_tokens)
        return None
    mm: Dict[str, Any] = {}
    is_vl = hasattr(br.runner.hf_config, "vision_config") and getattr(br.runner.model, "visual", None) is not None
    if is_vl and (args.image_path is not None or getattr(args, "synthetic_image", False)):
        image = load_image(args.image_path) if args.image_path is not None else None
        ids, pix, grid = make_multimodal_inputs(hf_config=br.runner.hf_config, batch_size=setting.batch_size,
                                                input_len=setting.input_len, image=image, seed=seed)
        setting = BenchSetting(setting.batch_size, ids.shape[1], setting.output_len)
        mm = {"pixel_values": pix.to(dev), "image_grid_thw": grid.to(dev), "benchmark_vision_timing": True}
        ids = ids.to(dev)
    else:
        ids = make_synthetic_input_ids(batch_size=setting.batch_size, input_len=setting.input_len,
                                       vocab_size=br.runner.vocab_size, seed=seed, device=dev)
    use_events = dev.type == "cuda"
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(setting.output_len + 1)] if use_events else []
    # --profile: one trace for the prefill and one for a window of decode steps (separate files, like the
    # stage switches of pymllm/bench_one_batch.py:668-758); NVTX ranges mark both stages for external tools
    import contextlib

    from .utils.profiling import nvtx_range, torch_profiler

    traces: List[str] = []
    tag = f"bs{setting.batch_size}_in{setting.input_len}_out{setting.output_len}"

    def stage_profiler(stage: str):
        on = bool(record_result and args.profile and args.profile_stage in ("all", stage))
        return torch_profiler(on, args.profile_activities, args.profile_record_shapes,
                              filename_prefix=args.profile_filename_prefix, tag=f"{tag}_{stage}", exported=traces)

    if use_events:
        _sync(dev)
        ev[0].record()
    with stage_profiler("prefill"), nvtx_range("bench_one_batch.prefill"):
        prefill_latency, nxt = _timed_call(dev, lambda: br.extend(ids, **mm))
    if use_events:
        ev[1].record()
    decode_lat: List[float] = []
    n_decode = setting.output_len - 1
    win_start = min(max(0, n_decode - 1), args.profile_start_step if args.profile_start_step is not None else n_decode // 2)
    win_end = min(n_decode, win_start + max(1, args.profile_steps))
    with contextlib.ExitStack() as window:
        for step in range(n_decode):
            if step == win_start:
                window.enter_context(stage_profiler("decode"))
            with nvtx_range("bench_one_batch.decode_step"):
                lat, nxt = _timed_call(dev, lambda: br.decode(nxt))
            if use_events:
                ev[step + 2].record()
            decode_lat.append(lat)
            if step + 1 == win_end:
                window.close()
            if args.log_decode_step and (step + 1) % args.log_decode_step == 0:
                logger.info("decode step %d: %.3f ms, %.1f tok/s", step + 1, lat * 1e3, setting.batch_size / lat)
    _sync(dev)
    extra: Dict[str, Any] = {"tp_size": pstate.get_tensor_model_parallel_world_size()}
    if traces:
        extra["profile_traces"] = list(traces)
    if mm:
        fb0 = br.last_forward_batch
        vit_ms, vit_tok = float(fb0.vit_prefill_ms or 0.0), int(fb0.vit_prefill_tokens or 0)
        extra.update(vit_prefill_ms=vit_ms, vit_prefill_tokens=vit_tok,
                     vit_prefill_tps=_safe_div(vit_tok, vit_ms / 1e3), llm_prefill_ms=float(fb0.llm_prefill_ms or 0.0),
                     multimodal_prefill_tps=_safe_div(setting.batch_size * setting.input_len, prefill_latency))
    if use_events:
        dp = ev[0].elapsed_time(ev[1]) / 1e3
        dd = [ev[i + 1].elapsed_time(ev[i + 2]) / 1e3 for i in range(setting.output_len - 1)]
        extra["device_prefill_latency"] = _max_over_ranks(dp, dev)
        extra["device_median_decode_latency"] = _max_over_ranks(statistics.median(dd) if dd else 0.0, dev)
    prefill_latency = _max_over_ranks(prefill_latency, dev)
    decode_lat = [_max_over_ranks(x, dev) for x in decode_lat] if pstate.get_tensor_model_parallel_world_size() > 1 else decode_lat
    row = summarize_latencies(setting=setting, prefill_latency=prefill_latency, decode_latencies=decode_lat,
                              run_name=args.run_name, device=str(dev), dtype=str(br.runner.dtype).replace("torch.", ""),
                              cuda_graph=br.runner.cuda_graph_runner is not None, extra=extra)
    from . import ops

    if dev.type == "cuda":
        ops.check_status(dev.index)
    if record_result:
        logger.info("bs=%d in=%d out=%d: prefill %.1f tok/s, decode %.1f tok/s (median %.3f ms/step)",
                    setting.batch_size, setting.input_len, setting.output_len, row["prefill_throughput"],
                    row["median_decode_throughput"], row["median_decode_latency"] * 1e3)
        return row
    return None


def align_runner_capacity_with_batch_sizes(cfg: GlobalConfig, args: BenchArgs) -> None:
    biggest = max(args.batch_size)
    if (cfg.server.max_running_requests or 1) < biggest:
        sc = cfg.server
        sc.max_running_requests = biggest


def run_correctness_test(bench_runner: BenchRunner, args: BenchArgs) -> List[List[int]]:
    """Greedy smoke run: prefill a short seeded prompt and decode 16 tokens; returns the ids."""
    br = bench_runner
    br.clear()
    ids = make_synthetic_input_ids(batch_size=1, input_len=16, vocab_size=br.runner.vocab_size, seed=args.seed)
    nxt = br.extend(ids)
    out = [int(nxt[0])]
    for _ in range(15):
        nxt = br.decode(nxt)
        out.append(int(nxt[0]))
    print("greedy ids:", out)
    return [out]


def run_benchmark(cfg: GlobalConfig, args: BenchArgs) -> List[Dict[str, Any]]:
    align_runner_capacity_with_batch_sizes(cfg, args)
    br = BenchRunner.create(cfg)
    if args.correctness_test:
        run_correctness_test(br, args)
        return []
    rank0 = pstate.get_tp_group().rank_in_group == 0
    settings = generate_settings(args)
    if not args.skip_warmup and settings:
        s0 = settings[0]
        warm = BenchSetting(s0.batch_size, s0.input_len, min(32, s0.output_len))
        run_single_setting(bench_runner=br, args=args, setting=warm, seed=args.seed, record_result=False)
    rows = []
    for s in settings:
        row = run_single_setting(bench_runner=br, args=args, setting=s, seed=args.seed, record_result=True)
        if row is not None:
            rows.append(row)
            if rank0:
                with open(args.result_filename, "a") as f:
                    f.write(json.dumps(row) + "\n")
    return rows


def main(argv: Optional[Sequence[str]] = None) -> None:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(message)s")
    cfg, args = parse_args(argv)
    rows = run_benchmark(cfg, args)
    if pstate.get_tp_group().rank_in_group == 0:
        for r in rows:
            print(json.dumps(r))


if __name__ == "__main__":
    main()

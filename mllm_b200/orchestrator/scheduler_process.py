"""Continuous-batching scheduler: one iteration of its loop is one forward pass.

Policy of pymllm/orchestrator/scheduler_process.py:662-736 (first come first served; prefill
before decode; admit while ``running < max_running_requests``, the KV budget and the prefill token
budget allow), extended with what the reference declares but does not implement: **chunked
prefill** (a prompt longer than ``chunked_prefill_size`` is prefilled over several passes) and
**mixed batches** (running requests ride along in a prefill pass as one-token rows, so decode does
not stall behind long prompts).  The class is plain host logic around
:class:`ModelRunnerProcess`; :func:`run_scheduler_process` wraps it in the ZMQ event loop used by
the multi-process engine, and the in-process engine drives it from a thread.

With tensor parallelism every rank runs the same scheduler on the same request stream (rank 0
receives requests and broadcasts them), so all ranks build identical batches without a per-step
metadata exchange.
"""

from __future__ import annotations

import logging
import time
from collections import deque
from dataclasses import dataclass
from typing import Any, Deque, Dict, List, Optional, Tuple

import torch

from ..configs import ServerConfig
from ..engine.io_struct import AbortReq, BatchTokenIDOutput, FlushCacheReq, SharedQueueNotice, TokenizedGenerateReqInput
from ..engine.sampling_params import SamplingParams
from .model_runner_process import KVAllocationError, ModelRunnerProcess, Req

from ..utils.profiling import nvtx_range
logger = logging.getLogger(__name__)


@dataclass
class SchedulerStats:
    num_prefill_batches: int = 0
    num_decode_batches: int = 0
    num_mixed_batches: int = 0
    prefill_tokens: int = 0
    cached_tokens: int = 0
    decode_tokens: int = 0
    finished: int = 0
    aborted: int = 0
    last_prefill_tok_s: float = 0.0
    last_decode_tok_s: float = 0.0


class Scheduler:
    def __init__(self, mrp: ModelRunnerProcess, server_config: ServerConfig, eos_token_ids: Optional[List[int]] = None,
                 enable_mixed: bool = True) -> None:
        self.mrp = mrp
        self.cfg = server_config
        self.eos_token_ids = set(eos_token_ids or [])
        self.enable_mixed = enable_mixed
        self.waiting: Deque[Req] = deque()
        self.prefilling: List[Req] = []   # admitted, prompt not fully computed yet
        self.running: List[Req] = []      # generating
        self.stats = SchedulerStats()
        self.max_running = server_config.max_running_requests or 1
        self.chunk = server_config.chunked_prefill_size
        self.max_prefill_tokens = server_config.max_prefill_tokens or 16384
        self.stream_interval = server_config.stream_interval
        self.context_len = mrp.runner.context_len
        self._decode_steps = 0
        self._stop_tokenizer = None       # built on the first request with stop strings

    # ------------------------------------------------------------------ intake
    def add_request(self, t: TokenizedGenerateReqInput) -> Optional[str]:
        """Queue a request. Returns an error string when it cannot be served at all."""
        try:
            sp = SamplingParams.from_dict(t.sampling_params)
        except (ValueError, TypeError) as exc:      # a malformed request must not end the serving loop
            return f"invalid sampling parameters: {exc}"
        ids = list(t.input_ids)
        if not ids:
            return "empty prompt"
        # an id outside the embedding table would be an out-of-bounds read on the device
        vocab = int(self.mrp.runner.vocab_size)
        lo, hi = min(ids), max(ids)
        if lo < 0 or hi >= vocab:
            return f"token id {lo if lo < 0 else hi} is outside the vocabulary (0..{vocab - 1})"
        if len(ids) >= self.context_len:
            ids = ids[: self.context_len - 1]
        sp.max_new_tokens = max(0, min(sp.max_new_tokens, self.context_len - len(ids)))
        if len(ids) + 1 > self.mrp.runner.max_total_num_tokens:
            return f"prompt of {len(ids)} tokens exceeds the KV pool ({self.mrp.runner.max_total_num_tokens} tokens)"
        # a request alone in the pool must be able to finish: prompt + output may not exceed the pool
        # (whole pages, one page kept back for the rounding of the last one)
        page = max(1, int(getattr(self.cfg, "radix_cache_page_size", 1) or 1))
        room = self.mrp.runner.max_total_num_tokens - (len(ids) + page - 1) // page * page - (page if page > 1 else 0)
        sp.max_new_tokens = max(1, min(sp.max_new_tokens, room)) if sp.max_new_tokens > 0 else 0
        if self.cfg.max_queued_requests is not None and len(self.waiting) >= self.cfg.max_queued_requests:
            return "queue full"
        bad = self._vision_inputs_error(ids, t.mm_inputs, len(ids) < len(t.input_ids))
        if bad:
            return bad
        if t.return_logprob and getattr(self.cfg, "pp_size", 1) > 1:
            return "log-probabilities are not available with pipeline parallelism (the logits live on the last stage)"
        stop_ids = set(sp.stop_token_ids or [])
        if not sp.ignore_eos:
            stop_ids |= self.eos_token_ids
        extra_key = None
        if t.mm_inputs and t.mm_inputs.get("image_hash"):
            extra_key = str(t.mm_inputs["image_hash"])
        req = Req(rid=t.rid, input_ids=ids, sampling=sp, stream=t.stream, input_text=t.input_text,
                  mm_inputs=t.mm_inputs, extra_key=extra_key, stop_token_ids=stop_ids,
                  created_time=t.created_time or time.time(), return_logprob=bool(t.return_logprob),
                  top_logprobs_num=max(0, min(int(t.top_logprobs_num or 0), vocab)), stop_strs=[s for s in (sp.stop or []) if s])
        if t.mm_inputs and "mrope_position_delta" in t.mm_inputs:
            req.mrope_delta = int(t.mm_inputs["mrope_position_delta"])
        self.waiting.append(req)
        return None

    def _vision_inputs_error(self, ids: List[int], mm: Optional[Dict[str, Any]], truncated: bool) -> Optional[str]:
        """Pixels, grids and vision tokens of a request must agree before it reaches the model: the vision tower
        writes one feature row per vision token, and a mismatch found there would end the serving loop."""
        if not mm or mm.get("pixel_values") is None or mm.get("image_grid_thw") is None:
            return None
        cfg = self.mrp.runner.hf_config
        image_id = getattr(cfg, "image_token_id", None)
        if image_id is None:
            return "this model takes no image or video inputs"
        if truncated:
            return "the prompt with its image / video tokens exceeds the context length"
        merge = int(getattr(getattr(cfg, "vision_config", None), "spatial_merge_size", 2) or 2)
        grids = mm["image_grid_thw"].reshape(-1, 3).tolist()
        rows = sum(int(t) * int(h) * int(w) for t, h, w in grids)
        want = sum(int(t) * (int(h) // merge) * (int(w) // merge) for t, h, w in grids)
        if int(mm["pixel_values"].shape[0]) != rows:
            return f"pixel_values has {int(mm['pixel_values'].shape[0])} rows, the grids describe {rows}"
        steps = mm.get("mrope_t_scale")
        if steps is not None and int(steps.numel()) != len(grids):
            return f"mrope_t_scale has {int(steps.numel())} entries for {len(grids)} grids"
        vision_ids = {image_id, getattr(cfg, "video_token_id", None)} - {None}
        have = sum(1 for tok in ids if tok in vision_ids)
        if have != want:
            return f"the prompt holds {have} image / video tokens, the grids describe {want}"
        return None

    def abort(self, rid: str) -> bool:
        for q in list(self.waiting):
            if q.rid == rid:
                self.waiting.remove(q)
                q.finished_reason = "abort"
                self.stats.aborted += 1
                return True
        for group in (self.prefilling, self.running):
            for q in group:
                if q.rid == rid and not q.finished:
                    q.finished_reason = "abort"
                    return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.prefilling or self.running)

    # ------------------------------------------------------------------ batch selection
    LPM_WINDOW = 64   # requests at the head of the queue that the prefix-aware policy looks at

    def _order_by_cached_prefix(self) -> None:
        """``schedule_policy == "lpm"``: among the first requests of the queue, those with the longest
        prefix already in the cache go first (they need the least new work and keep that prefix hot);
        ties keep their arrival order."""
        if len(self.waiting) < 2:
            return
        from ..mem_cache import RadixKey

        head = [self.waiting.popleft() for _ in range(min(self.LPM_WINDOW, len(self.waiting)))]
        cache = self.mrp.prefix_cache
        hit = {}
        for q in head:
            if q.mm_inputs and q.mm_inputs.get("pixel_values") is not None:
                hit[id(q)] = 0
            else:
                hit[id(q)] = cache.match_prefix(RadixKey(q.input_ids[: max(0, len(q.input_ids) - 1)], q.extra_key)).prefix_len
        head.sort(key=lambda q: -hit[id(q)])           # stable: arrival order among equals
        self.waiting.extendleft(reversed(head))

    def _admit_waiting(self) -> None:
        """Move requests from the queue into `prefilling` while the budgets allow."""
        if self.cfg.schedule_policy == "lpm" and len(self.running) + len(self.prefilling) < self.max_running:
            self._order_by_cached_prefix()
        while self.waiting:
            if len(self.running) + len(self.prefilling) >= self.max_running:
                break
            req = self.waiting[0]
            # conservative KV budget: the whole prompt plus its generation must fit beside what is reserved
            reserved = sum(q.sampling.max_new_tokens - len(q.output_ids) for q in self.running) + \
                sum(len(q.input_ids) - q.num_computed + q.sampling.max_new_tokens for q in self.prefilling)
            need = len(req.input_ids) + req.sampling.max_new_tokens
            budget = self.mrp.available_tokens() / self.cfg.schedule_conservativeness
            if self.mrp.free_req_slots() == 0 or (need + reserved > budget and (self.running or self.prefilling)):
                break
            self.waiting.popleft()
            try:
                self.mrp.admit(req)
            except KVAllocationError:
                self.waiting.appendleft(req)
                break
            self.stats.cached_tokens += req.cached_tokens
            self.prefilling.append(req)

    def get_next_batch_to_run(self) -> Tuple[str, List[Tuple[Req, int]]]:
        """("extend" | "decode" | "idle", rows).  Extend rows: (request, new tokens in this pass)."""
        self._sweep_finished()
        self._admit_waiting()
        if self.prefilling:
            rows: List[Tuple[Req, int]] = []
            budget = min(self.max_prefill_tokens, self.chunk or self.max_prefill_tokens)
            for req in self.prefilling:
                if budget <= 0:
                    break
                n = min(len(req.input_ids) - req.num_computed, budget)
                if req.mm_inputs and req.mm_inputs.get("pixel_values") is not None and req.num_computed == 0:
                    # the vision tower needs every image token of the prompt in one pass: no chunking
                    n = len(req.input_ids)
                if n > 0:
                    rows.append((req, n))
                    budget -= n
            if self.enable_mixed and self.running:
                rows.extend((q, 1) for q in self.running)
            return "extend", rows
        if self.running:
            return "decode", [(q, 1) for q in self.running]
        return "idle", []

    # ------------------------------------------------------------------ one iteration
    def step(self) -> Optional[BatchTokenIDOutput]:
        kind, rows = self.get_next_batch_to_run()
        if kind == "idle":
            return None
        t0 = time.perf_counter()
        try:
            # one named range per pass (visible in timeline tools next to the kernels it launched)
            with nvtx_range(f"scheduler.{kind}[{len(rows)}]"):
                if kind == "extend":
                    next_ids, produced, _ = self.mrp.extend(rows)
                    reqs = [rows[i][0] for i in produced]
                else:
                    reqs = [q for q, _ in rows]
                    next_ids, _ = self.mrp.decode(reqs)
        except KVAllocationError as exc:
            return self._shed_load(str(exc))
        with nvtx_range("scheduler.read_tokens"):
            ids = next_ids.tolist() if next_ids is not None and len(reqs) else []  # the step's one device->host sync
        dt = time.perf_counter() - t0
        now = time.time()
        n_prefill = sum(n for q, n in rows if q in self.prefilling) if kind == "extend" else 0
        if kind == "extend":
            mixed = any(q in self.running for q, _ in rows)
            self.stats.num_mixed_batches += int(mixed)
            self.stats.num_prefill_batches += 1
            self.stats.prefill_tokens += n_prefill
            self.stats.last_prefill_tok_s = n_prefill / dt if dt > 0 else 0.0
            if self.cfg.log_level in ("debug", "info"):
                logger.info("Prefill batch: #new-token %d, #cached-token %d, #running %d, #queue %d, input tok/s %.1f",
                            n_prefill, sum(q.cached_tokens for q, _ in rows if q in self.prefilling),
                            len(self.running), len(self.waiting), self.stats.last_prefill_tok_s)
        else:
            self.stats.num_decode_batches += 1
            self._decode_steps += 1
            self.stats.last_decode_tok_s = len(reqs) / dt if dt > 0 else 0.0
            iv = self.cfg.decode_log_interval
            if iv and self._decode_steps % iv == 0:
                logger.info("Decode batch: #running %d, #token %d, gen tok/s %.1f, #queue %d", len(self.running),
                            sum(q.seq_len for q in self.running), self.stats.last_decode_tok_s, len(self.waiting))
        for req, tok in zip(reqs, ids):
            if req.finished:  # aborted while the pass ran
                continue
            req.output_ids.append(int(tok))
            self.stats.decode_tokens += 1
            if len(req.output_ids) == 1:
                req.first_token_time = now
            self._check_finished(req, now)
        # prompts that completed their prefill start generating
        still = []
        for q in self.prefilling:
            if q.finished:
                still.append(q)          # finished on its first token (or aborted): the next sweep releases it
            elif q.num_computed >= len(q.input_ids):
                self.running.append(q)
            else:
                still.append(q)
        self.prefilling = still
        return self._collect_output(reqs)

    def _hits_stop_string(self, req: Req) -> bool:
        """Decodes the tail of the generated ids (long enough to hold the longest stop string that could
        have been completed by the newest token) and looks for the stop strings in it.  The detokenizer
        cuts the text at the match; here the request only has to stop."""
        if self._stop_tokenizer is None:
            from ..utils.tokenizer import get_tokenizer

            sc = self.cfg
            self._stop_tokenizer = get_tokenizer(sc.tokenizer_path, self.mrp.runner.vocab_size, sc.tokenizer_mode,
                                                 sc.trust_remote_code)
        window = max(len(s) for s in req.stop_strs) + 8      # a token holds at least one byte of text
        tail = self._stop_tokenizer.decode(req.output_ids[-window:], skip_special_tokens=req.sampling.skip_special_tokens)
        return any(s in tail for s in req.stop_strs)

    def _check_finished(self, req: Req, now: float) -> None:
        tok = req.output_ids[-1]
        if tok in req.stop_token_ids:
            req.finished_reason = "stop"
        elif req.stop_strs and self._hits_stop_string(req):
            req.finished_reason = "stop"
        elif len(req.output_ids) >= req.sampling.max_new_tokens:
            req.finished_reason = "length"
        elif req.seq_len >= self.context_len:
            req.finished_reason = "length"
        if req.finished:
            req.finish_time = now

    def _sweep_finished(self) -> None:
        for group_name in ("running", "prefilling"):
            group = getattr(self, group_name)
            keep = []
            for q in group:
                if q.finished:
                    self.mrp.release(q, cache=q.finished_reason != "abort")
                    if q.finished_reason == "abort":
                        self.stats.aborted += 1
                    else:
                        self.stats.finished += 1
                else:
                    keep.append(q)
            setattr(self, group_name, keep)

    def _shed_load(self, why: str, requeue_lone: bool = False) -> Optional[BatchTokenIDOutput]:
        """The pool ran dry mid-flight: retract the youngest running request back to the queue.  A request
        that holds the pool alone is ended instead (``requeue_lone`` queues it again all the same)."""
        logger.warning("KV allocation failed (%s); retracting a request", why)
        victims = self.prefilling or self.running
        if not victims:
            raise RuntimeError(why)
        q = victims[-1]
        alone = len(self.prefilling) + len(self.running) == 1
        (self.prefilling if q in self.prefilling else self.running).remove(q)
        if alone and not requeue_lone:
            # nobody else holds KV: queueing it again would meet the same full pool for ever
            q.finished_reason = "length"
            q.finish_time = time.time()
            self.mrp.release(q, cache=True)
            self.stats.finished += 1
            return self._collect_output([q])
        self.mrp.release(q, cache=True)
        if q.mm_inputs:
            # the whole prompt is prefilled again: pixels are needed again and positions start over
            q.mm_inputs.pop("_consumed", None)
            q.mrope_delta = int(q.mm_inputs.get("mrope_position_delta", 0))
        q.input_ids = q.all_ids()
        q.sampling.max_new_tokens = max(0, q.sampling.max_new_tokens - len(q.output_ids))
        retained, q.output_ids = q.output_ids, []
        q.num_computed = q.prefix_len = 0
        q.__dict__.setdefault("_retained", []).extend(retained)
        self.waiting.appendleft(q)
        return None

    def _collect_output(self, reqs: List[Req]) -> Optional[BatchTokenIDOutput]:
        out = BatchTokenIDOutput([], [], [], [], [], [])
        for q in reqs:
            if not q.output_ids and not q.finished:
                continue
            due = q.finished or (q.stream and len(q.output_ids) - q.last_stream_len >= self.stream_interval)
            if not due:
                continue
            q.last_stream_len = len(q.output_ids)
            prior = q.__dict__.get("_retained", [])
            out.rids.append(q.rid)
            out.finished_reasons.append(q.finished_reason)
            out.output_ids.append(prior + list(q.output_ids))
            out.skip_special_tokens.append(q.sampling.skip_special_tokens)
            out.stop_strs.append(list(q.stop_strs) or None)
            out.prompt_tokens.append(len(q.input_ids) - len(prior))
            out.completion_tokens.append(len(prior) + len(q.output_ids))
            out.cached_tokens.append(q.cached_tokens)
            timing = None
            if q.finished:
                ttft = max(0.0, q.first_token_time - q.created_time)
                n = len(q.output_ids)
                tpot = (q.finish_time - q.first_token_time) / (n - 1) if n > 1 else 0.0
                timing = {"ttft_s": ttft, "tpot_s": tpot, "e2e_s": q.finish_time - q.created_time}
            out.timing.append(timing)
            out.logprobs.append({"token_logprobs": list(q.output_logprobs), "top_logprobs": list(q.output_top_logprobs)}
                                if q.return_logprob else None)
        return out if out.rids else None

    def abort_outputs(self, rids: List[str]) -> BatchTokenIDOutput:
        return BatchTokenIDOutput(rids, ["abort"] * len(rids), [[] for _ in rids], [True] * len(rids), [0] * len(rids),
                                  [0] * len(rids), [0] * len(rids), [None] * len(rids))

    def flush_cache(self) -> bool:
        if self.has_work():
            return False
        return self.mrp.flush_cache()


# ----------------------------------------------------------------------------------------------
# process wrapper (multi-process engine): ZMQ in from the tokenizer, ZMQ out to the detokenizer
# ----------------------------------------------------------------------------------------------
def build_scheduler(server_config: ServerConfig, hf_config=None, quantization_method=None, kv_cache_dtype="auto",
                    device: Optional[str] = None, eos_token_ids: Optional[List[int]] = None) -> Scheduler:
    import os

    from ..executor import ModelRunner
    from ..parallel import state as pstate

    if server_config.world_size > 1:
        pstate.init_distributed()
        if not pstate.model_parallel_is_initialized():
            pstate.initialize_model_parallel(tp_size=server_config.tp_size, ep_size=server_config.ep_size,
                                              pp_size=server_config.pp_size)
    gpu = server_config.base_gpu_id + int(os.environ.get("LOCAL_RANK", "0"))
    runner = ModelRunner(server_config, hf_config=hf_config, gpu_id=gpu, quantization_method=quantization_method,
                         kv_cache_dtype=kv_cache_dtype, device=device)
    runner.initialize()
    if eos_token_ids is None:
        eos_token_ids = resolve_eos_token_ids(runner.hf_config, server_config.model_path, server_config.tokenizer_path)
    mrp = ModelRunnerProcess(runner, disable_radix_cache=server_config.disable_radix_cache)
    return Scheduler(mrp, server_config, eos_token_ids)


def _eos_list(eos) -> List[int]:
    if isinstance(eos, bool) or eos is None:
        return []
    if isinstance(eos, int):
        return [eos]
    return [int(e) for e in eos if isinstance(e, int) and not isinstance(e, bool)] if isinstance(eos, (list, tuple)) else []


def resolve_eos_token_ids(hf_config, model_path=None, tokenizer_path=None) -> List[int]:
    """End-of-sequence ids in the reference's order of precedence (pymllm/engine/launch.py:57-107): the config, its
    ``text_config`` (vision-language checkpoints), ``generation_config.json`` beside the checkpoint (many chat
    checkpoints list several ids there), then the tokenizer's own id."""
    import json
    import os

    for cfg in (hf_config, getattr(hf_config, "text_config", None)):
        ids = _eos_list(getattr(cfg, "eos_token_id", None)) if cfg is not None else []
        if ids:
            return ids
    local = None if model_path is None or str(model_path).startswith("preset:") else str(model_path)
    if local is not None and os.path.isfile(os.path.join(local, "generation_config.json")):
        try:
            with open(os.path.join(local, "generation_config.json")) as f:
                ids = _eos_list(json.load(f).get("eos_token_id"))
            if ids:
                return ids
        except (OSError, ValueError):
            pass
    tok_path = tokenizer_path if tokenizer_path is not None else model_path
    if tok_path is not None and not str(tok_path).startswith("preset:") and any(
            os.path.isfile(os.path.join(str(tok_path), f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        try:
            from ..utils.tokenizer import get_tokenizer

            eos = getattr(get_tokenizer(str(tok_path), 0), "eos_token_id", None)
            return _eos_list(eos)
        except Exception:  # a checkpoint without tokenizer files: no id from here
            pass
    return []


def run_scheduler_process(server_config: ServerConfig, recv_addr: Optional[str], send_addr: Optional[str], pipe_writer=None,
                          hf_config=None, quantization_method=None, kv_cache_dtype: str = "auto",
                          device: Optional[str] = None, rank: int = 0, world_size: int = 1,
                          master_port: Optional[int] = None, tensor_queue=None) -> None:
    """Event loop: receive -> schedule -> forward -> stream out (one forward per iteration).

    With ``world_size > 1`` one such process runs per rank.  Rank 0 owns the sockets; at the top of
    every iteration it hands the messages it received to the other ranks (object broadcast over a gloo
    group, never over the GPU), so every rank applies the same requests in the same order and the
    schedulers stay in lock step without exchanging batch metadata.  Only rank 0 answers."""
    import os

    import zmq

    from .ipc_utils import make_socket, setup_subprocess_logging

    setup_subprocess_logging(server_config.log_level)
    if world_size > 1:
        os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world_size), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(master_port or 29577))
    try:
        sched = build_scheduler(server_config, hf_config, quantization_method, kv_cache_dtype, device)
        ctrl = None
        if world_size > 1:
            import torch.distributed as dist

            ctrl = dist.new_group(backend="gloo")  # host-side control plane
    except Exception as exc:  # readiness handshake carries the failure to the parent
        if pipe_writer is not None:
            pipe_writer.send({"status": "error", "error": repr(exc)})
        raise
    ctx = zmq.Context()
    recv = send = poller = None
    if rank == 0:
        recv = make_socket(ctx, zmq.PULL, recv_addr, bind=False)
        send = make_socket(ctx, zmq.PUSH, send_addr, bind=True)
        poller = zmq.Poller()
        poller.register(recv, zmq.POLLIN)
    if pipe_writer is not None:
        pipe_writer.send({"status": "ready", "max_total_num_tokens": sched.mrp.runner.max_total_num_tokens})
    try:
        scheduler_event_loop(sched, recv, send, poller, rank, world_size, ctrl, tensor_queue if rank == 0 else None)
    finally:
        if world_size > 1:   # leave the process groups in an orderly way: their worker threads must not outlive main
            import torch.distributed as dist

            try:
                if dist.is_initialized():
                    dist.destroy_process_group()
            except Exception:
                pass


def _take_from_shared_queue(tensor_queue, notice):
    """The request announced by ``notice``: its metadata from shared memory, its tensors from the queue."""
    import queue as _queue

    if tensor_queue is None:
        return {"error": "request body was sent through a shared-memory queue this scheduler does not have", "rid": notice.rid}
    try:
        rid, meta, mm = tensor_queue.get(timeout=30)
    except _queue.Empty:
        return {"error": "shared-memory queue: announced request never arrived", "rid": notice.rid}
    meta.mm_inputs = mm
    return meta


def scheduler_event_loop(sched: "Scheduler", recv, send, poller, rank: int = 0, world_size: int = 1, ctrl_group=None,
                         tensor_queue=None) -> None:
    idle_ms = 1000 if world_size == 1 else 50  # followers wait in the broadcast: keep the heartbeat short
    while True:
        msgs: Optional[list] = None
        if rank == 0:
            msgs = []
            # drain the inbox; sleep on the socket when there is nothing to run
            timeout = 0 if sched.has_work() else idle_ms
            while dict(poller.poll(timeout)):
                m = recv.recv_pyobj()
                if isinstance(m, SharedQueueNotice):
                    m = _take_from_shared_queue(tensor_queue, m)
                    if isinstance(m, dict):  # could not be fetched: answer, do not hand on to the other ranks
                        send.send_pyobj(m)
                        continue
                msgs.append(m)
                timeout = 0
        if world_size > 1:
            import torch.distributed as dist

            box = [msgs]
            dist.broadcast_object_list(box, src=0, group=ctrl_group)
            msgs = box[0]
        for msg in msgs:
            if msg is None:
                if rank == 0 and send is not None:
                    send.send_pyobj(None)  # lets the detokenizer count this replica out
                return
            if isinstance(msg, TokenizedGenerateReqInput):
                try:
                    err = sched.add_request(msg)
                except Exception as exc:  # every rank sees the same message, so every rank refuses it alike
                    logger.exception("request %s refused at intake", getattr(msg, "rid", "?"))
                    err = f"request refused: {type(exc).__name__}: {exc}"
                if err is not None and rank == 0:
                    send.send_pyobj({"error": err, "rid": msg.rid})
            elif isinstance(msg, AbortReq):
                if sched.abort(msg.rid) and rank == 0:
                    send.send_pyobj(sched.abort_outputs([msg.rid]))
            elif isinstance(msg, FlushCacheReq):
                ok = sched.flush_cache()
                if rank == 0:
                    send.send_pyobj({"flush_cache": ok})
        out = sched.step()
        if out is not None and rank == 0:
            send.send_pyobj(out)

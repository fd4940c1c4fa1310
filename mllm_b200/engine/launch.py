"""Engine: the object a program (or the HTTP server) talks to.

Public surface of pymllm/engine/launch.py:130-658 — ``launch()``, ``generate()``,
``generate_async()``, ``shutdown()``, ``is_healthy`` — over two deployments:

* ``mode="multiproc"`` (the reference's layout): tokenizer, scheduler(+GPU) and detokenizer run
  as spawned daemon processes connected by ZMQ ``ipc://`` sockets; each child reports
  ``{"status": "ready"}`` on a pipe; a health thread polls ``is_alive`` every 5 s.
* ``mode="inproc"``: the same three workers run inside this process, the scheduler loop on a
  thread.  No serialisation on the hot path; used by tests, benchmarks and single-GPU embedding.

Both deliver results through :class:`RequestResponseProcess`, so streaming, abort and
back-pressure behave identically.
"""

from __future__ import annotations

import asyncio
import copy
import logging
import multiprocessing as mp
import os
import threading
import time
import uuid
from typing import Any, AsyncIterator, Dict, Iterator, List, Optional, Union

from ..configs import GlobalConfig, ServerConfig, get_global_config
from ..orchestrator.request_response_process import ReqState, RequestResponseProcess
from .io_struct import AbortReq, FlushCacheReq, GenerateReqInput

logger = logging.getLogger(__name__)
DEFAULT_MAX_NEW_TOKENS = 128


def model_default_max_new_tokens(hf_config) -> Optional[int]:
    """The output-length limit a checkpoint's config declares (``max_new_tokens`` / ``max_tokens`` /
    ``max_completion_tokens``, as pymllm/engine/launch.py:110-127), used when a request gives none."""
    for cfg in (hf_config, getattr(hf_config, "text_config", None)):
        for name in ("max_new_tokens", "max_tokens", "max_completion_tokens"):
            v = getattr(cfg, name, None) if cfg is not None else None
            if isinstance(v, int) and not isinstance(v, bool) and v > 0:
                return v
    return None


def _free_port() -> int:
    import socket

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return int(sk.getsockname()[1])


class Engine:
    def __init__(self, config: Optional[Union[GlobalConfig, ServerConfig]] = None, mode: str = "inproc",
                 hf_config: Any = None, device: Optional[str] = None) -> None:
        if config is None:
            config = get_global_config()
        if isinstance(config, GlobalConfig):
            self.server_config = config.server
            self.quant_method = config.quantization.method
            self.kv_cache_dtype = config.quantization.kv_cache_dtype
        else:
            self.server_config = config
            self.quant_method, self.kv_cache_dtype = None, "auto"
        if mode not in ("inproc", "multiproc"):
            raise ValueError("mode must be 'inproc' or 'multiproc'")
        self._resolve_paths()
        self.mode = mode
        self.hf_config = hf_config
        self.device = device
        self._launched = False
        self._healthy = False
        self._procs: List[mp.Process] = []
        self._threads: List[threading.Thread] = []
        self._stop = threading.Event()
        self.rr: Optional[RequestResponseProcess] = None
        self.scheduler = None
        self._addrs: List[str] = []

    def _resolve_paths(self) -> None:
        """A model path that is neither a directory nor a preset names a hub repository: fetch it once, before any
        process is started, and point the model and tokenizer paths at the local snapshot."""
        from ..utils.hub import resolve_model_path

        sc = self.server_config
        if sc.model_path is None:
            return
        same_tokenizer = sc.tokenizer_path is None or str(sc.tokenizer_path) == str(sc.model_path)
        local = resolve_model_path(sc.model_path, sc.download_dir)
        if str(local) != str(sc.model_path):
            sc.model_path = local
        if same_tokenizer:
            sc.tokenizer_path = sc.model_path
        else:
            sc.tokenizer_path = resolve_model_path(sc.tokenizer_path, sc.download_dir)

    # ------------------------------------------------------------------ lifecycle
    def launch(self) -> "Engine":
        if self._launched:
            return self
        logging.getLogger("mllm_b200").setLevel(getattr(logging, self.server_config.log_level.upper(), logging.INFO))
        if self.mode == "inproc" and (self.server_config.dp_size > 1 or self.server_config.world_size > 1):
            raise ValueError("tensor / data parallel engines run as processes: use mode='multiproc'")
        if self.mode == "inproc":
            self._launch_inproc()
        else:
            self._launch_processes()
        self._launched = self._healthy = True
        return self

    def _vocab_size(self) -> int:
        from ..executor import load_hf_config, text_config_of

        if self.hf_config is None:
            self.hf_config = load_hf_config(self.server_config.model_path)
        self._default_max_new_tokens = model_default_max_new_tokens(self.hf_config) or DEFAULT_MAX_NEW_TOKENS
        return int(getattr(text_config_of(self.hf_config), "vocab_size", 1024))

    def _mm_config(self):
        """Vision-token ids and patch geometry for the tokenizer's built-in image path (None: text model)."""
        cfg = self.hf_config
        vc = getattr(cfg, "vision_config", None)
        if vc is None or getattr(cfg, "image_token_id", None) is None:
            return None
        from ..utils.image_processor import CLIP_MEAN, CLIP_STD

        family = str(getattr(cfg, "model_type", ""))
        clip = family in ("qwen2_vl", "qwen2_5_vl")                 # these normalise with CLIP statistics
        video = None if getattr(cfg, "video_token_id", None) is None else int(cfg.video_token_id)
        # Qwen3-VL prompts hold one timestamped block per temporal patch; Qwen2-VL / Qwen2.5-VL prompts hold one
        # block per clip, and Qwen2.5-VL advances the temporal position by seconds x tokens_per_second
        layout = "clip" if clip else "frames"
        tps = float(getattr(vc, "tokens_per_second", 2)) if family == "qwen2_5_vl" else None
        return dict(video_token_id=video, video_layout=layout, tokens_per_second=tps,
                    image_mean=list(CLIP_MEAN) if clip else 0.5, image_std=list(CLIP_STD) if clip else 0.5,
                    image_token_id=int(cfg.image_token_id), vision_start_token_id=int(cfg.vision_start_token_id),
                    vision_end_token_id=int(getattr(cfg, "vision_end_token_id", cfg.vision_start_token_id)),
                    patch_size=int(vc.patch_size), merge_size=int(getattr(vc, "spatial_merge_size", 2)),
                    temporal_patch_size=int(getattr(vc, "temporal_patch_size", 2)))

    def _launch_inproc(self) -> None:
        from ..orchestrator.detokenizer_process import DetokenizerWorker
        from ..orchestrator.scheduler_process import build_scheduler
        from ..orchestrator.tokenizer_process import TokenizerWorker

        sc = self.server_config
        vocab = self._vocab_size()
        self.tokenizer_worker = TokenizerWorker(sc.tokenizer_path, sc.context_length, vocab, sc.tokenizer_mode,
                                                sc.trust_remote_code, self._mm_config())
        self.detokenizer_worker = DetokenizerWorker(sc.tokenizer_path, vocab, sc.tokenizer_mode, sc.trust_remote_code)
        self.scheduler = build_scheduler(sc, self.hf_config, self.quant_method, self.kv_cache_dtype, self.device)
        tok = self.tokenizer_worker.tokenizer
        if getattr(tok, "eos_token_id", None) is not None and not self.scheduler.eos_token_ids:
            self.scheduler.eos_token_ids = {int(tok.eos_token_id)}
        self._inbox: List[Any] = []
        self._inbox_lock = threading.Lock()
        self._wake = threading.Event()
        self.rr = RequestResponseProcess(self._inproc_send, sc.max_queued_requests)
        t = threading.Thread(target=self._inproc_loop, name="mllm_b200-scheduler", daemon=True)
        t.start()
        self._threads.append(t)

    def _inproc_send(self, msg: Any) -> None:
        with self._inbox_lock:
            self._inbox.append(msg)
        self._wake.set()

    def _inproc_loop(self) -> None:
        import torch

        sched = self.scheduler
        if sched.mrp.device.type == "cuda":
            torch.cuda.set_device(sched.mrp.device)
        try:
            while not self._stop.is_set():
                with self._inbox_lock:
                    msgs, self._inbox = self._inbox, []
                for m in msgs:
                    if isinstance(m, AbortReq):
                        if sched.abort(m.rid):
                            self.rr.handle_output(self.detokenizer_worker.detokenize(sched.abort_outputs([m.rid])))
                    elif isinstance(m, FlushCacheReq):
                        sched.flush_cache()
                    else:
                        try:
                            err = sched.add_request(self.tokenizer_worker.tokenize(m))
                        except Exception as exc:  # bad request: report, keep serving
                            err = f"{type(exc).__name__}: {exc}"
                        if err is not None:
                            self.rr.handle_output({"error": err, "rid": m["rid"]})
                if not sched.has_work():
                    self._wake.wait(timeout=0.5)
                    self._wake.clear()
                    continue
                out = sched.step()
                if out is not None:
                    self.rr.handle_output(self.detokenizer_worker.detokenize(out))
        except Exception:
            logger.exception("scheduler loop died")
            self._healthy = False

    def _launch_processes(self) -> None:
        import zmq

        from ..orchestrator.detokenizer_process import run_detokenizer_process
        from ..orchestrator.ipc_utils import make_ipc_address, make_socket
        from ..orchestrator.scheduler_process import run_scheduler_process
        from ..orchestrator.tokenizer_process import run_tokenizer_process

        sc = self.server_config
        vocab = self._vocab_size()
        uid = f"{os.getpid()}_{uuid.uuid4().hex[:8]}"
        world, replicas = sc.world_size, max(1, int(sc.dp_size))
        a_rr_tok, a_detok_rr = make_ipc_address("rr_tok", uid), make_ipc_address("detok_rr", uid)
        a_tok_sched = [make_ipc_address(f"tok_sched{r}", uid) for r in range(replicas)]
        a_sched_detok = [make_ipc_address(f"sched_detok{r}", uid) for r in range(replicas)]
        self._addrs = [a_rr_tok, a_detok_rr, *a_tok_sched, *a_sched_detok]
        ctx = mp.get_context("spawn")
        pipes = []

        def spawn(target, kwargs):
            r, w = ctx.Pipe(duplex=False)
            p = ctx.Process(target=target, kwargs=dict(kwargs, pipe_writer=w), daemon=True)
            p.start()
            self._procs.append(p)
            pipes.append((p, r))

        self._zmq = zmq.Context()
        self._to_tok = make_socket(self._zmq, zmq.PUSH, a_rr_tok, bind=True)
        # shared-memory fast path for requests that carry tensors (images): one queue per replica,
        # handed to the tokenizer (writer) and to the replica's rank 0 (reader) at spawn time
        self._tensor_queues = None
        if sc.enable_shared_queue:
            from ..orchestrator.shared_memory_queue import TensorQueue

            self._tensor_queues = [TensorQueue(transport_mode=sc.tensor_transport_mode, ctx=ctx) for _ in range(replicas)]
        spawn(run_tokenizer_process, dict(tokenizer_path=sc.tokenizer_path, recv_addr=a_rr_tok, send_addr=a_tok_sched,
                                          context_length=sc.context_length, vocab_size=vocab,
                                          tokenizer_mode=sc.tokenizer_mode, trust_remote_code=sc.trust_remote_code,
                                          log_level=sc.log_level, mm_config=self._mm_config(),
                                          shared_queues=self._tensor_queues))
        # data parallelism: `dp_size` complete replicas (each `world` GPUs wide) behind the tokenizer's
        # router; replica r uses GPUs base + r * world ... base + (r + 1) * world - 1
        for rep in range(replicas):
            rsc = copy.copy(sc)
            rsc.base_gpu_id = sc.base_gpu_id + rep * world
            port = _free_port() if world > 1 else None
            for rank in range(world):  # one scheduler + model runner per GPU; rank 0 owns the sockets
                spawn(run_scheduler_process, dict(server_config=rsc, recv_addr=a_tok_sched[rep] if rank == 0 else None,
                                                  send_addr=a_sched_detok[rep] if rank == 0 else None,
                                                  hf_config=self.hf_config, quantization_method=self.quant_method,
                                                  kv_cache_dtype=self.kv_cache_dtype, device=self.device, rank=rank,
                                                  world_size=world, master_port=port,
                                                  tensor_queue=self._tensor_queues[rep] if self._tensor_queues and rank == 0 else None))
        spawn(run_detokenizer_process, dict(tokenizer_path=sc.tokenizer_path, recv_addr=a_sched_detok,
                                            send_addr=a_detok_rr, vocab_size=vocab, tokenizer_mode=sc.tokenizer_mode,
                                            trust_remote_code=sc.trust_remote_code, log_level=sc.log_level))
        for p, r in pipes:  # readiness handshake; EOF or an error message fails the launch
            try:
                if not r.poll(600):
                    raise RuntimeError(f"process {p.name} did not become ready")
                msg = r.recv()
            except EOFError as exc:
                raise RuntimeError(f"process {p.name} exited during start-up") from exc
            if msg.get("status") != "ready":
                raise RuntimeError(f"process {p.name} failed to start: {msg}")
        self._from_detok = make_socket(self._zmq, zmq.PULL, a_detok_rr, bind=False)
        self._send_lock = threading.Lock()

        def send(msg):
            with self._send_lock:
                self._to_tok.send_pyobj(msg)

        self.rr = RequestResponseProcess(send, sc.max_queued_requests)
        t = threading.Thread(target=self._recv_loop, name="mllm_b200-recv", daemon=True)
        t.start()
        h = threading.Thread(target=self._health_loop, name="mllm_b200-health", daemon=True)
        h.start()
        self._threads += [t, h]

    def _recv_loop(self) -> None:
        import zmq

        poller = zmq.Poller()
        poller.register(self._from_detok, zmq.POLLIN)
        while not self._stop.is_set():
            if dict(poller.poll(200)):
                self.rr.handle_output(self._from_detok.recv_pyobj())

    def _health_loop(self) -> None:
        while not self._stop.wait(5.0):
            if any(not p.is_alive() for p in self._procs):
                self._healthy = False
            self.rr.gc()

    @property
    def is_healthy(self) -> bool:
        return self._launched and self._healthy and not self._stop.is_set()

    def shutdown(self) -> None:
        if not self._launched:
            return
        self._stop.set()
        if self.mode == "inproc":
            self._wake.set()
            for t in self._threads:
                t.join(timeout=10)
            if self.scheduler is not None:
                self.scheduler.mrp.runner.shutdown()
        else:
            try:
                self._to_tok.send_pyobj(None)
            except Exception:
                pass
            for p in self._procs:
                p.join(timeout=5)
                if p.is_alive():
                    p.terminate()
                    p.join(timeout=2)
                if p.is_alive():
                    p.kill()
                    p.join(timeout=2)
            for t in self._threads:
                t.join(timeout=2)
            try:
                self._zmq.destroy(linger=0)
            except Exception:
                pass
            from ..orchestrator.ipc_utils import cleanup_ipc

            cleanup_ipc(self._addrs)
            for q in getattr(self, "_tensor_queues", None) or []:
                try:
                    q.close()
                except Exception:
                    pass
        self._launched = self._healthy = False

    # ------------------------------------------------------------------ requests
    def _submit(self, obj: GenerateReqInput) -> List[tuple]:
        obj.normalize_batch_and_arguments()
        out = []
        for i in range(obj.batch_size):
            one = obj[i]
            sp = dict(one.sampling_params or {})
            sp.setdefault("max_new_tokens", sp.pop("max_tokens", getattr(self, "_default_max_new_tokens", DEFAULT_MAX_NEW_TOKENS)))
            req = one.to_request_dict()
            req["sampling_params"] = sp
            req["rid"] = one.rid
            req["created_time"] = time.time()
            out.append((one.rid, self.rr.add_request(req)))
        return out

    @staticmethod
    def _final(rid: str, st: ReqState) -> Dict[str, Any]:
        if st.error is not None:
            raise ValueError(st.error)
        last = st.out_list[-1]
        meta = {"finish_reason": last["finish_reason"], "prompt_tokens": last["prompt_tokens"],
                "completion_tokens": last["completion_tokens"], "cached_tokens": last["cached_tokens"],
                "timing": last["timing"]}
        if last.get("logprobs") is not None:
            meta["output_token_logprobs"] = last["logprobs"]
        return {"rid": rid, "text": last["text"], "output_ids": last["output_ids"], "meta_info": meta}

    def generate(self, prompt: Optional[Union[str, List[str]]] = None, sampling_params=None, input_ids=None,
                 image_data=None, stream: bool = False, rid=None, timeout: Optional[float] = None,
                 return_logprob: bool = False, top_logprobs_num: int = 0, video_data=None):
        """Blocking generation. One prompt -> dict, a list -> list of dicts; ``stream=True`` (single
        prompt) returns an iterator of incremental dicts with a ``delta`` field.  With ``return_logprob``
        ``meta_info["output_token_logprobs"]`` holds the log-probability (and text) of every generated token
        and, per token, the ``top_logprobs_num`` most likely alternatives.  ``video_data``: frames of a clip (array
        ``[F, H, W, 3]``, list of images, ``.npy`` file, or ``{"frames": ..., "fps": f}``) for the model families with
        video tokens."""
        obj = GenerateReqInput(rid=rid, text=prompt, input_ids=input_ids, sampling_params=sampling_params,
                               image_data=image_data, video_data=video_data, stream=stream, return_logprob=return_logprob or None,
                               top_logprobs_num=top_logprobs_num or None)
        subs = self._submit(obj)
        if stream:
            if len(subs) != 1:
                raise ValueError("stream=True takes a single prompt")
            return self._stream_sync(*subs[0], timeout)
        results = []
        for r, st in subs:
            deadline = None if timeout is None else time.time() + timeout
            while not st.finished:
                st.event.wait(0.05 if deadline is None else max(0.0, min(0.05, deadline - time.time())))
                st.event.clear()
                if not self.is_healthy:
                    raise RuntimeError("engine is not healthy")
                if deadline is not None and time.time() > deadline:
                    self.rr.abort(r)
                    raise TimeoutError(f"request {r} timed out")
            try:
                results.append(self._final(r, st))
            finally:
                self.rr.pop(r)
        return results[0] if obj.is_single else results

    # ---- conversation helpers (roles of ARGeneration::chat / perfSummary in the reference's C++ runtime) ----
    def _chat_tokenizer(self):
        tok = getattr(self, "_chat_tok", None)
        if tok is None:
            w = getattr(self, "tokenizer_worker", None)
            if w is not None:
                tok = w.tokenizer
            else:
                from ..utils.tokenizer import get_tokenizer

                sc = self.server_config
                tok = get_tokenizer(sc.tokenizer_path, self._vocab_size(), sc.tokenizer_mode, sc.trust_remote_code)
            self._chat_tok = tok
        return tok

    def chat(self, messages: List[Dict[str, Any]], sampling_params=None, stream: bool = False, tools=None,
             image_data=None, timeout: Optional[float] = None, video_data=None, **template_kwargs):
        """Renders ``messages`` (``[{"role": ..., "content": ...}, ...]``) with the tokenizer's chat template
        (ChatML when it has none) and generates the assistant turn; same return types as ``generate``."""
        from ..utils.tokenizer import render_chatml

        tok = self._chat_tokenizer()
        prompt = None
        if getattr(tok, "chat_template", None):
            try:
                prompt = tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=True, tools=tools,
                                                 **template_kwargs)
            except Exception as exc:
                logger.warning("chat template failed (%s); using ChatML", exc)
        if prompt is None:
            prompt = render_chatml(messages, add_generation_prompt=True)
        return self.generate(prompt, sampling_params, image_data=image_data, stream=stream, timeout=timeout,
                             video_data=video_data)

    @staticmethod
    def perf_summary(result: Dict[str, Any]) -> Dict[str, float]:
        """Time to first token and prefill / decode rates of one finished request, from its timing record."""
        meta = result["meta_info"]
        t = meta.get("timing") or {}
        p, c = meta.get("prompt_tokens", 0), meta.get("completion_tokens", 0)
        ttft, tpot, e2e = t.get("ttft_s", 0.0), t.get("tpot_s", 0.0), t.get("e2e_s", 0.0)
        return {"ttft_ms": ttft * 1e3, "tpot_ms": tpot * 1e3, "e2e_ms": e2e * 1e3,
                "prefill_tokens": p, "cached_tokens": meta.get("cached_tokens", 0), "decode_tokens": c,
                "prefill_tokens_per_s": p / ttft if ttft > 0 else 0.0,
                "decode_tokens_per_s": 1.0 / tpot if tpot > 0 else 0.0}

    def _stream_sync(self, rid: str, st: ReqState, timeout) -> Iterator[Dict[str, Any]]:
        sent = 0
        try:
            while True:
                st.event.wait(0.05)
                st.event.clear()
                if st.error is not None:
                    raise ValueError(st.error)
                while sent < len(st.out_list):
                    o = st.out_list[sent]
                    sent += 1
                    yield {"rid": rid, "text": o["text"], "delta": o["delta"], "output_ids": o["output_ids"],
                           "meta_info": {k: o[k] for k in ("finish_reason", "prompt_tokens", "completion_tokens",
                                                           "cached_tokens", "timing")}}
                if st.finished and sent >= len(st.out_list):
                    return
                if not self.is_healthy:
                    raise RuntimeError("engine is not healthy")
        finally:
            if not st.finished:
                self.rr.abort(rid)
            self.rr.pop(rid)

    async def generate_async(self, obj: GenerateReqInput) -> AsyncIterator[Dict[str, Any]]:
        """Async generation for the HTTP layer: yields incremental dicts when ``obj.stream`` else the
        final dict of every request of the batch.  Cancelling the consumer aborts the request."""
        subs = self._submit(obj)
        loop = asyncio.get_running_loop()
        for rid, st in subs:
            sent = 0
            try:
                while True:
                    await loop.run_in_executor(None, st.event.wait, 0.05)
                    st.event.clear()
                    if st.error is not None:
                        raise ValueError(st.error)
                    if obj.stream:
                        while sent < len(st.out_list):
                            o = st.out_list[sent]
                            sent += 1
                            yield {"rid": rid, "text": o["text"], "delta": o["delta"], "output_ids": o["output_ids"],
                                   "meta_info": {k: o[k] for k in ("finish_reason", "prompt_tokens",
                                                                   "completion_tokens", "cached_tokens", "timing")}}
                    if st.finished and (not obj.stream or sent >= len(st.out_list)):
                        if not obj.stream:
                            yield self._final(rid, st)
                        break
                    if not self.is_healthy:
                        raise RuntimeError("engine is not healthy")
            finally:
                if not st.finished:
                    self.rr.abort(rid)
                self.rr.pop(rid)

    def abort(self, rid: str) -> None:
        self.rr.abort(rid)

    def flush_cache(self) -> None:
        self.rr._send(FlushCacheReq())

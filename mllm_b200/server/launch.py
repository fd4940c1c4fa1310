"""OpenAI-compatible HTTP server.

Endpoints and behaviour of pymllm/server/launch.py:120-1190: ``GET /health``, ``/health_generate``,
``/model_info``, ``/server_info``, ``/v1/models``, ``/v1/models/{id}``; ``POST /generate``,
``/v1/completions``, ``/v1/chat/completions``, ``/flush_cache``, ``/abort_request``; Bearer-token
auth on everything but the health routes; chat-template rendering with a ChatML fallback; SSE
streaming (``data: {...}\\n\\n`` ... ``data: [DONE]``) that aborts the request when the client goes
away; ``stream_options.include_usage``; reasoning and tool-call parsing for whole replies and for
streams; an optional ``debug_timing`` block; error mapping 400 / 401 / 429 / 500 / 503.
Additions: ``/metrics`` (Prometheus text, behind ``--server.enable_metrics``) and ``/flush_cache``
actually flushes the prefix cache when the engine is idle.

    python -m mllm_b200.server.launch --server.model_path /path/to/model --server.port 30000
"""

from __future__ import annotations

import asyncio
import json
import logging
import time
import uuid
from typing import Any, AsyncIterator, Dict, List, Optional, Union

from fastapi import FastAPI, Request
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse
from pydantic import BaseModel, Field

from ..configs import GlobalConfig, get_global_config, make_args, read_args
from ..engine.io_struct import GenerateReqInput
from ..engine.launch import Engine
from ..parsers import ReasoningParser, ToolCallParser
from ..utils.metrics import Metrics
from ..utils.tokenizer import render_chatml

logger = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------------
# request schemas
# ------------------------------------------------------------------------------------------
class GenerateRequest(BaseModel):
    text: Optional[Union[str, List[str]]] = None
    input_ids: Optional[Union[List[int], List[List[int]]]] = None
    sampling_params: Optional[Union[Dict[str, Any], List[Dict[str, Any]]]] = None
    image_data: Optional[Any] = None
    stream: bool = False
    rid: Optional[Union[str, List[str]]] = None
    return_logprob: Optional[bool] = None
    top_logprobs_num: Optional[int] = None
    # carried for request-format compatibility; not acted on
    logprob_start_len: Optional[int] = None
    video_data: Optional[Any] = None
    audio_data: Optional[Any] = None
    lora_path: Optional[str] = None
    session_params: Optional[Dict[str, Any]] = None


class StreamOptions(BaseModel):
    include_usage: bool = False
    continuous_usage_stats: Optional[bool] = False   # usage so far in every streamed chunk


class CompletionRequest(BaseModel):
    model: Optional[str] = None
    prompt: Union[str, List[str], List[int]]
    max_tokens: Optional[int] = 16
    temperature: Optional[float] = 1.0
    top_p: Optional[float] = 1.0
    top_k: Optional[int] = -1
    min_p: Optional[float] = 0.0
    n: int = 1
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    stop: Optional[Union[str, List[str]]] = None
    stop_token_ids: Optional[List[int]] = None
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    user: Optional[str] = None
    logprobs: Optional[int] = None
    echo: bool = False
    ignore_eos: bool = False


class ChatMessage(BaseModel):
    role: str
    content: Optional[Union[str, List[Dict[str, Any]]]] = None
    name: Optional[str] = None
    tool_calls: Optional[List[Dict[str, Any]]] = None
    tool_call_id: Optional[str] = None


class ChatCompletionRequest(BaseModel):
    model: Optional[str] = None
    messages: List[ChatMessage]
    max_tokens: Optional[int] = None
    max_completion_tokens: Optional[int] = None
    temperature: Optional[float] = 1.0
    top_p: Optional[float] = 1.0
    top_k: Optional[int] = -1
    min_p: Optional[float] = 0.0
    n: int = 1
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    stop: Optional[Union[str, List[str]]] = None
    stop_token_ids: Optional[List[int]] = None
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    logprobs: Optional[bool] = None
    top_logprobs: Optional[int] = None
    tools: Optional[List[Dict[str, Any]]] = None
    tool_choice: Optional[Any] = None
    separate_reasoning: bool = True
    stream_reasoning: bool = True     # False: reasoning text is delivered in one piece when the thinking block ends
    user: Optional[str] = None
    chat_template_kwargs: Optional[Dict[str, Any]] = None
    ignore_eos: bool = False


class AbortRequest(BaseModel):
    rid: str


def _error(status: int, message: str, err_type: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse(status_code=status, content={"error": {"message": message, "type": err_type, "code": status}})


def _sampling(req, default_max: int) -> Dict[str, Any]:
    max_new = getattr(req, "max_completion_tokens", None) or req.max_tokens or default_max
    return {
        "max_new_tokens": max_new, "temperature": req.temperature if req.temperature is not None else 1.0,
        "top_p": req.top_p if req.top_p is not None else 1.0, "top_k": req.top_k if req.top_k else -1,
        "min_p": req.min_p or 0.0, "stop": req.stop, "stop_token_ids": req.stop_token_ids,
        "frequency_penalty": req.frequency_penalty, "presence_penalty": req.presence_penalty,
        "repetition_penalty": req.repetition_penalty, "seed": req.seed, "ignore_eos": req.ignore_eos,
    }


def _extract_images(messages: List[ChatMessage]) -> List[Any]:
    images = []
    for m in messages:
        if isinstance(m.content, list):
            for part in m.content:
                if part.get("type") == "image_url":
                    url = part.get("image_url")
                    images.append(url.get("url") if isinstance(url, dict) else url)
                elif part.get("type") == "image":
                    images.append(part.get("image"))
    return images


def _extract_videos(messages: List[ChatMessage]) -> List[Any]:
    """Video parts in order: ``{"type": "video", "video": <frames | .npy file | container file | {"frames": ...,
    "fps": f}>}`` or ``{"type": "video_url", "video_url": {"url": <container file | data:video/...;base64,...>}}``."""
    videos = []
    for m in messages:
        if isinstance(m.content, list):
            for part in m.content:
                if part.get("type") == "video":
                    videos.append(part.get("video"))
                elif part.get("type") == "video_url":
                    url = part.get("video_url")
                    url = url.get("url") if isinstance(url, dict) else url
                    videos.append(url[len("file://"):] if isinstance(url, str) and url.startswith("file://") else url)
    return videos


def messages_to_prompt(tokenizer, messages: List[ChatMessage], tools=None, template_kwargs=None) -> str:
    """Chat template of the tokenizer when it has one, else ChatML.  Image parts become the
    Qwen-VL placeholder ``<|vision_start|><|image_pad|><|vision_end|>``."""
    plain = []
    for m in messages:
        d = {k: v for k, v in m.model_dump().items() if v is not None}
        if isinstance(m.content, list):
            text = ""
            for part in m.content:
                if part.get("type") == "text":
                    text += part.get("text", "")
                elif part.get("type") in ("image_url", "image"):
                    text += "<|vision_start|><|image_pad|><|vision_end|>"
                elif part.get("type") in ("video", "video_url"):
                    text += "<|vision_start|><|video_pad|><|vision_end|>"
            d["content"] = text
        plain.append(d)
    if getattr(tokenizer, "chat_template", None):
        try:
            return tokenizer.apply_chat_template(plain, tokenize=False, add_generation_prompt=True, tools=tools,
                                                 **(template_kwargs or {}))
        except Exception as exc:
            logger.warning("chat template failed (%s); using ChatML", exc)
    return render_chatml(plain, add_generation_prompt=True)


def _n_sampling(sp: Dict[str, Any], n: int, prompts: int) -> List[Dict[str, Any]]:
    """``n`` samples per prompt: the same parameters, with distinct seeds when one was given (otherwise the
    sampler draws a fresh seed per request anyway)."""
    out = []
    for _ in range(prompts):
        for j in range(n):
            d = dict(sp)
            if d.get("seed") is not None:
                d["seed"] = int(d["seed"]) + j
            out.append(d)
    return out


def _usage(meta: Dict[str, Any]) -> Dict[str, Any]:
    p, c = meta.get("prompt_tokens", 0), meta.get("completion_tokens", 0)
    return {"prompt_tokens": p, "completion_tokens": c, "total_tokens": p + c,
            "prompt_tokens_details": {"cached_tokens": meta.get("cached_tokens", 0)}}


def _chat_logprobs(lp: Optional[Dict[str, Any]]) -> Optional[Dict[str, Any]]:
    """Chat-completions layout: one entry per generated token with its alternatives."""
    if lp is None:
        return None

    def entry(tok: str, val: float) -> Dict[str, Any]:
        return {"token": tok, "logprob": val, "bytes": list(tok.encode("utf-8"))}

    content = []
    for i, val in enumerate(lp["token_logprobs"]):
        e = entry(lp["tokens"][i], val)
        e["top_logprobs"] = [entry(t, v) for t, (_, v) in zip(lp["top_tokens"][i], lp["top_logprobs"][i])]
        content.append(e)
    return {"content": content}


def _completion_logprobs(lp: Optional[Dict[str, Any]]) -> Optional[Dict[str, Any]]:
    """Legacy completions layout: parallel lists plus character offsets into the returned text."""
    if lp is None:
        return None
    offsets, pos = [], 0
    for t in lp["tokens"]:
        offsets.append(pos)
        pos += len(t)
    tops = [{t: v for t, (_, v) in zip(lp["top_tokens"][i], lp["top_logprobs"][i])} or None
            for i in range(len(lp["token_logprobs"]))]
    return {"tokens": lp["tokens"], "token_logprobs": lp["token_logprobs"], "top_logprobs": tops, "text_offset": offsets}


def _debug_timing(meta: Dict[str, Any]) -> Optional[Dict[str, Any]]:
    t = meta.get("timing")
    if not t:
        return None
    c = meta.get("completion_tokens", 0)
    return {"ttft_ms": t["ttft_s"] * 1e3, "tpot_ms": t["tpot_s"] * 1e3, "e2e_ms": t["e2e_s"] * 1e3,
            "prefill_tokens": meta.get("prompt_tokens", 0), "cached_tokens": meta.get("cached_tokens", 0),
            "decode_tokens": c, "decode_tokens_per_s": (c - 1) / (t["tpot_s"] * (c - 1)) if c > 1 and t["tpot_s"] > 0 else 0.0}


async def _watch_disconnect(request: Request, agen: AsyncIterator[Any]) -> AsyncIterator[Any]:
    """Relay ``agen`` and stop (which aborts the request in the engine) once the client is gone."""
    it = agen.__aiter__()
    try:
        while True:
            nxt = asyncio.ensure_future(it.__anext__())
            while not nxt.done():
                done, _ = await asyncio.wait({nxt}, timeout=1.0)
                if not done and await request.is_disconnected():
                    nxt.cancel()
                    return
            try:
                yield nxt.result()
            except StopAsyncIteration:
                return
    finally:
        await agen.aclose()


# ------------------------------------------------------------------------------------------
def create_app(engine: Engine, cfg: Optional[GlobalConfig] = None) -> FastAPI:
    cfg = cfg or get_global_config()
    sc = engine.server_config
    app = FastAPI(title="mllm_b200", root_path=sc.fastapi_root_path or "")
    app.add_middleware(CORSMiddleware, allow_origins=sc.cors_allow_origins, allow_methods=["*"], allow_headers=["*"])
    metrics = Metrics(enabled=sc.enable_metrics)
    model_name = sc.served_model_name or str(sc.model_path)
    created = int(time.time())

    def tokenizer():
        w = getattr(engine, "tokenizer_worker", None)
        if w is None:
            from ..utils.tokenizer import get_tokenizer

            engine.tokenizer_worker = type("W", (), {"tokenizer": get_tokenizer(sc.tokenizer_path)})()
            w = engine.tokenizer_worker
        return w.tokenizer

    @app.middleware("http")
    async def auth(request: Request, call_next):
        path = request.url.path
        if sc.api_key and not path.startswith("/health") and request.method != "OPTIONS":
            given = request.headers.get("authorization", "")
            allowed = {f"Bearer {sc.api_key}"} | ({f"Bearer {sc.admin_api_key}"} if sc.admin_api_key else set())
            if given not in allowed:
                return _error(401, "Invalid or missing API key", "authentication_error")
        t0 = time.perf_counter()
        resp = await call_next(request)
        metrics.observe_http(path, resp.status_code, time.perf_counter() - t0)
        return resp

    @app.get("/health")
    async def health():
        return JSONResponse({"status": "ok"}) if engine.is_healthy else JSONResponse({"status": "unhealthy"}, 503)

    @app.get("/health_generate")
    async def health_generate():
        if not engine.is_healthy:
            return JSONResponse({"status": "unhealthy"}, 503)
        obj = GenerateReqInput(text="ping", sampling_params={"max_new_tokens": 1, "temperature": 0.0})
        try:
            async for _ in engine.generate_async(obj):
                pass
        except Exception as exc:
            return JSONResponse({"status": "unhealthy", "error": str(exc)}, 503)
        return {"status": "ok"}

    @app.get("/model_info")
    async def model_info():
        return {"model_path": str(sc.model_path), "tokenizer_path": str(sc.tokenizer_path), "is_generation": True,
                "served_model_name": model_name}

    @app.get("/server_info")
    async def server_info():
        import dataclasses

        d = {k: (str(v) if not isinstance(v, (int, float, bool, type(None), list, dict)) else v)
             for k, v in dataclasses.asdict(sc).items() if "api_key" not in k}
        return {"server": d, "quantization": {"method": cfg.quantization.method,
                                              "kv_cache_dtype": cfg.quantization.kv_cache_dtype}}

    @app.get("/v1/models")
    async def list_models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": created, "owned_by": "mllm_b200"}]}

    @app.get("/v1/models/{model_id:path}")
    async def get_model(model_id: str):
        if model_id != model_name:
            return _error(404, f"model {model_id!r} not found", "not_found_error")
        return {"id": model_name, "object": "model", "created": created, "owned_by": "mllm_b200"}

    @app.get("/metrics")
    async def prometheus():
        if not sc.enable_metrics:
            return _error(404, "metrics are disabled; start with --server.enable_metrics", "not_found_error")
        sched = getattr(engine, "scheduler", None)
        if sched is not None:
            metrics.sample_scheduler(sched)
        return PlainTextResponse(metrics.render(), media_type="text/plain; version=0.0.4")

    @app.api_route("/flush_cache", methods=["GET", "POST"])
    async def flush_cache():
        engine.flush_cache()
        return {"status": "requested"}

    @app.post("/abort_request")
    async def abort_request(body: AbortRequest):
        engine.abort(body.rid)
        return {"status": "ok", "rid": body.rid}

    async def _collect(obj: GenerateReqInput) -> List[Dict[str, Any]]:
        outs = []
        async for o in engine.generate_async(obj):
            outs.append(o)
        for o in outs:
            metrics.observe_request(o["meta_info"])
        return outs

    def _map_exc(exc: Exception) -> JSONResponse:
        if isinstance(exc, RuntimeError) and "queue is full" in str(exc):
            return _error(429, str(exc), "rate_limit_error")
        if isinstance(exc, (ValueError, KeyError)):
            return _error(400, str(exc))
        if isinstance(exc, RuntimeError) and "not healthy" in str(exc):
            return _error(503, str(exc), "service_unavailable")
        logger.exception("request failed")
        return _error(500, f"{type(exc).__name__}: {exc}", "internal_error")

    # ---------------------------------------------------------------- /generate
    @app.api_route("/generate", methods=["POST", "PUT"])
    async def generate(body: GenerateRequest, request: Request):
        obj = GenerateReqInput(rid=body.rid, text=body.text, input_ids=body.input_ids, sampling_params=body.sampling_params,
                               image_data=body.image_data, video_data=body.video_data, stream=body.stream,
                               return_logprob=body.return_logprob or None, top_logprobs_num=body.top_logprobs_num or None)
        if body.stream:
            async def sse():
                try:
                    async for o in _watch_disconnect(request, engine.generate_async(obj)):
                        yield f"data: {json.dumps(o)}\n\n"
                except Exception as exc:
                    yield f"data: {json.dumps({'error': str(exc)})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        try:
            outs = await _collect(obj)
        except Exception as exc:
            return _map_exc(exc)
        return outs[0] if obj.is_single else outs

    # ---------------------------------------------------------------- /v1/completions
    @app.post("/v1/completions")
    async def completions(body: CompletionRequest, request: Request):
        n = int(body.n or 1)
        if not 1 <= n <= 16 or (n > 1 and body.stream):
            return _error(400, "n must be between 1 and 16, and 1 when streaming")
        want_lp = body.logprobs is not None
        if want_lp and body.stream:
            return _error(400, "logprobs are not supported together with stream")
        if want_lp and not 0 <= int(body.logprobs) <= 20:
            return _error(400, "logprobs must be between 0 and 20")
        if body.echo and body.stream:
            return _error(400, "echo is not supported together with stream")
        sp = _sampling(body, 16)
        kw: Dict[str, Any] = {}
        prompts: List[Any]
        if isinstance(body.prompt, list) and body.prompt and isinstance(body.prompt[0], int):
            prompts = [body.prompt]
            kw["input_ids"] = prompts[0] if n == 1 else [p for p in prompts for _ in range(n)]
        else:
            prompts = body.prompt if isinstance(body.prompt, list) else [body.prompt]
            kw["text"] = body.prompt if n == 1 else [p for p in prompts for _ in range(n)]
        sps: Any = sp if n == 1 else _n_sampling(sp, n, len(prompts))
        obj = GenerateReqInput(sampling_params=sps, stream=body.stream, return_logprob=True if want_lp else None,
                               top_logprobs_num=int(body.logprobs) if want_lp and body.logprobs else None, **kw)
        cid = f"cmpl-{uuid.uuid4().hex}"
        if body.stream:
            include_usage = bool(body.stream_options and body.stream_options.include_usage)

            async def sse():
                meta = {}
                try:
                    async for o in _watch_disconnect(request, engine.generate_async(obj)):
                        meta = o["meta_info"]
                        chunk = {"id": cid, "object": "text_completion", "created": int(time.time()), "model": model_name,
                                 "choices": [{"index": 0, "text": o["delta"], "finish_reason": meta["finish_reason"]}]}
                        yield f"data: {json.dumps(chunk)}\n\n"
                    if include_usage and meta:
                        yield "data: " + json.dumps({"id": cid, "object": "text_completion", "created": int(time.time()),
                                                     "model": model_name, "choices": [], "usage": _usage(meta)}) + "\n\n"
                    if meta:
                        metrics.observe_request(meta)
                except Exception as exc:
                    yield f"data: {json.dumps({'error': {'message': str(exc)}})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        try:
            outs = await _collect(obj)
        except Exception as exc:
            return _map_exc(exc)
        total = {"prompt_tokens": 0, "completion_tokens": 0, "cached_tokens": 0}
        choices = []
        for i, o in enumerate(outs):
            for k in total:
                total[k] += o["meta_info"].get(k, 0)
            text = o["text"]
            if body.echo:   # choices come prompt-major: n per prompt
                p = prompts[i // n]
                text = (p if isinstance(p, str) else tokenizer().decode(p)) + text
            choices.append({"index": i, "text": text, "finish_reason": o["meta_info"]["finish_reason"],
                            "logprobs": _completion_logprobs(o["meta_info"].get("output_token_logprobs"))})
        resp = {"id": cid, "object": "text_completion", "created": int(time.time()), "model": model_name,
                "choices": choices, "usage": _usage(total)}
        if sc.enable_debug_timing and outs:
            resp["debug_timing"] = _debug_timing(outs[-1]["meta_info"])
        return resp

    # ---------------------------------------------------------------- /v1/chat/completions
    @app.post("/v1/chat/completions")
    async def chat_completions(body: ChatCompletionRequest, request: Request):
        n = int(body.n or 1)
        if not 1 <= n <= 16 or (n > 1 and body.stream):
            return _error(400, "n must be between 1 and 16, and 1 when streaming")
        if body.logprobs and body.stream:
            return _error(400, "logprobs are not supported together with stream")
        if body.top_logprobs is not None and not (body.logprobs and 0 <= body.top_logprobs <= 20):
            return _error(400, "top_logprobs needs logprobs=true and a value between 0 and 20")
        try:
            prompt = messages_to_prompt(tokenizer(), body.messages, body.tools, body.chat_template_kwargs)
        except Exception as exc:
            return _error(400, f"could not render the chat template: {exc}")
        images = _extract_images(body.messages)
        videos = _extract_videos(body.messages)
        sp = _sampling(body, 128)
        obj = GenerateReqInput(text=prompt if n == 1 else [prompt] * n, sampling_params=sp if n == 1 else _n_sampling(sp, n, 1),
                               stream=body.stream, image_data=(images or None) if n == 1 else ([images] * n if images else None),
                               video_data=(videos or None) if n == 1 else ([videos] * n if videos else None),
                               return_logprob=True if body.logprobs else None, top_logprobs_num=body.top_logprobs or None)
        cid = f"chatcmpl-{uuid.uuid4().hex}"
        use_reasoning = bool(sc.reasoning_parser) and body.separate_reasoning
        use_tools = bool(sc.tool_call_parser) and bool(body.tools)
        if body.stream:
            include_usage = bool(body.stream_options and body.stream_options.include_usage)

            async def sse():
                rp = ReasoningParser(sc.reasoning_parser, stream_reasoning=body.stream_reasoning) if use_reasoning else None
                every = bool(body.stream_options and body.stream_options.continuous_usage_stats)
                tp = ToolCallParser(sc.tool_call_parser, body.tools) if use_tools else None
                meta: Dict[str, Any] = {}
                saw_tool = False

                def chunk(delta: Dict[str, Any], finish=None) -> str:
                    d = {"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model_name,
                         "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
                    if every and meta:
                        d["usage"] = _usage(meta)
                    return "data: " + json.dumps(d) + "\n\n"
                try:
                    yield chunk({"role": "assistant", "content": ""})
                    async for o in _watch_disconnect(request, engine.generate_async(obj)):
                        meta = o["meta_info"]
                        text = o["delta"]
                        reasoning = ""
                        if rp is not None:
                            reasoning, text = rp.parse_stream_chunk(text)
                        if reasoning:
                            yield chunk({"reasoning_content": reasoning})
                        calls = []
                        if tp is not None:
                            text, calls = tp.parse_stream_chunk(text)
                            if meta["finish_reason"] is not None:
                                calls += tp.flush()
                        if text:
                            yield chunk({"content": text})
                        for c in calls:
                            saw_tool = True
                            yield chunk({"tool_calls": [c.to_openai_dict(streaming=True)]})
                        if meta["finish_reason"] is not None:
                            fin = "tool_calls" if saw_tool and meta["finish_reason"] == "stop" else meta["finish_reason"]
                            yield chunk({}, fin)
                    if include_usage and meta:
                        yield "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": int(time.time()),
                                                     "model": model_name, "choices": [], "usage": _usage(meta)}) + "\n\n"
                    if meta:
                        metrics.observe_request(meta)
                except Exception as exc:
                    yield f"data: {json.dumps({'error': {'message': str(exc)}})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        try:
            outs = await _collect(obj)
        except Exception as exc:
            return _map_exc(exc)
        choices = []
        total = {"prompt_tokens": 0, "completion_tokens": 0, "cached_tokens": 0}
        for i, o in enumerate(outs):
            for k in total:
                total[k] += o["meta_info"].get(k, 0)
            text = o["text"]
            message: Dict[str, Any] = {"role": "assistant"}
            if use_reasoning:
                reasoning, text = ReasoningParser(sc.reasoning_parser).parse_non_stream(text)
                message["reasoning_content"] = reasoning
            finish = o["meta_info"]["finish_reason"]
            if use_tools:
                text, calls = ToolCallParser(sc.tool_call_parser, body.tools).parse_non_stream(text)
                if calls:
                    message["tool_calls"] = [c.to_openai_dict(streaming=False) for c in calls]
                    if finish == "stop":
                        finish = "tool_calls"
            message["content"] = text
            choices.append({"index": i, "message": message, "finish_reason": finish,
                            "logprobs": _chat_logprobs(o["meta_info"].get("output_token_logprobs"))})
        o = outs[-1]
        resp = {"id": cid, "object": "chat.completion", "created": int(time.time()), "model": model_name,
                "choices": choices, "usage": _usage(total if n > 1 else o["meta_info"])}
        if sc.enable_debug_timing:
            resp["debug_timing"] = _debug_timing(o["meta_info"])
        return resp

    return app


def launch_server(argv=None) -> None:
    import uvicorn

    parser = make_args()
    parser.add_argument("--engine-mode", choices=["inproc", "multiproc"], default="multiproc")
    ns, _ = parser.parse_known_args(argv)
    cfg = read_args(argv, parser)
    logging.basicConfig(level=getattr(logging, cfg.server.log_level.upper(), logging.INFO))
    engine = Engine(cfg, mode=ns.engine_mode).launch()
    app = create_app(engine, cfg)
    try:
        loop = "uvloop"
        try:
            import uvloop  # noqa: F401
        except ImportError:
            loop = "asyncio"
        uvicorn.run(app, host=cfg.server.host, port=cfg.server.port, log_level=cfg.server.log_level, loop=loop,
                    timeout_keep_alive=5)
    finally:
        engine.shutdown()


def main() -> None:
    launch_server()


if __name__ == "__main__":
    main()

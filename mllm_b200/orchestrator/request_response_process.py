"""Front-end bridge living in the main process (role of
pymllm/orchestrator/request_response_process.py:29-236): keeps one ``ReqState`` per request id,
applies queue back-pressure (``max_queued_requests`` -> RuntimeError -> HTTP 429), fans results out
to waiting coroutines / threads, turns aborts into messages and drops stale states."""

from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

from ..engine.io_struct import AbortReq, BatchStrOutput

STALE_SECONDS = 30 * 60


@dataclass
class ReqState:
    out_list: List[Dict[str, Any]] = field(default_factory=list)
    event: threading.Event = field(default_factory=threading.Event)
    finished: bool = False
    created: float = field(default_factory=time.time)
    error: Optional[str] = None


class RequestResponseProcess:
    def __init__(self, send_fn: Callable[[Any], None], max_queued_requests: Optional[int] = None) -> None:
        self._send = send_fn
        self.max_queued = max_queued_requests
        self.states: Dict[str, ReqState] = {}
        self.lock = threading.Lock()

    def add_request(self, req: Dict[str, Any]) -> ReqState:
        with self.lock:
            live = sum(1 for s in self.states.values() if not s.finished)
            if self.max_queued is not None and live >= self.max_queued:
                raise RuntimeError(f"request queue is full ({live} >= {self.max_queued})")
            st = ReqState()
            self.states[req["rid"]] = st
        self._send(req)
        return st

    def abort(self, rid: str) -> None:
        self._send(AbortReq(rid=rid))

    def handle_output(self, msg: Any) -> None:
        """Called by the receive loop with whatever the detokenizer sent."""
        if isinstance(msg, BatchStrOutput):
            for i, rid in enumerate(msg.rids):
                st = self.states.get(rid)
                if st is None:
                    continue
                st.out_list.append({
                    "text": msg.output_strs[i], "delta": msg.deltas[i], "output_ids": msg.output_ids[i],
                    "finish_reason": msg.finished_reasons[i], "prompt_tokens": msg.prompt_tokens[i],
                    "completion_tokens": msg.completion_tokens[i],
                    "cached_tokens": msg.cached_tokens[i] if msg.cached_tokens else 0,
                    "timing": msg.timing[i] if msg.timing else None,
                    "logprobs": msg.logprobs[i] if msg.logprobs else None,
                })
                if msg.finished_reasons[i] is not None:
                    st.finished = True
                st.event.set()
        elif isinstance(msg, dict) and "error" in msg:
            st = self.states.get(msg.get("rid", ""))
            if st is not None:
                st.error, st.finished = msg["error"], True
                st.event.set()

    def pop(self, rid: str) -> None:
        with self.lock:
            self.states.pop(rid, None)

    def gc(self) -> int:
        now = time.time()
        with self.lock:
            stale = [r for r, s in self.states.items() if now - s.created > STALE_SECONDS]
            for r in stale:
                del self.states[r]
        return len(stale)

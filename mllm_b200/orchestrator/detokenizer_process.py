"""Detokenizer worker (role of pymllm/orchestrator/detokenizer_process.py:20-233): decodes the full
list of generated ids of every request on every message and emits the text added since the
previous message (``delta``); incomplete UTF-8 tails are held back until they complete."""

from __future__ import annotations

import logging
from typing import Dict, Optional

from ..engine.io_struct import BatchStrOutput, BatchTokenIDOutput
from ..utils.tokenizer import get_tokenizer

logger = logging.getLogger(__name__)


class DetokenizerWorker:
    def __init__(self, tokenizer_path, vocab_size: int = 1024, tokenizer_mode: str = "auto",
                 trust_remote_code: bool = False) -> None:
        self.tokenizer = get_tokenizer(tokenizer_path, vocab_size, tokenizer_mode, trust_remote_code)
        self.sent: Dict[str, str] = {}

    def detokenize(self, batch: BatchTokenIDOutput) -> BatchStrOutput:
        out = BatchStrOutput([], [], [], [], [], [], [], [], [], [])
        for i, rid in enumerate(batch.rids):
            ids = batch.output_ids[i]
            text = self.tokenizer.decode(ids, skip_special_tokens=batch.skip_special_tokens[i]) if ids else ""
            finished = batch.finished_reasons[i]
            if finished is None and text.endswith("�"):
                text = text.rstrip("�")  # an incomplete multi-byte character: wait for the rest
            stops = batch.stop_strs[i] if batch.stop_strs else None
            if stops:
                # cut at the earliest stop string; while the request runs, hold back a tail that could
                # still turn into one, so that no part of a stop string is ever streamed
                cut = min((p for p in (text.find(s) for s in stops) if p >= 0), default=-1)
                if cut >= 0:
                    text = text[:cut]
                elif finished is None:
                    keep = len(text) - (max(len(s) for s in stops) - 1)
                    text = text[: max(len(self.sent.get(rid, "")), keep, 0)]
            prev = self.sent.get(rid, "")
            delta = text[len(prev):] if text.startswith(prev) else text
            if finished is None:
                self.sent[rid] = text
            else:
                self.sent.pop(rid, None)
            out.rids.append(rid)
            out.finished_reasons.append(finished)
            out.output_strs.append(text)
            out.deltas.append(delta)
            out.output_ids.append(ids)
            out.prompt_tokens.append(batch.prompt_tokens[i])
            out.completion_tokens.append(batch.completion_tokens[i])
            out.cached_tokens.append(batch.cached_tokens[i] if batch.cached_tokens else 0)
            out.timing.append(batch.timing[i] if batch.timing else None)
            lp = batch.logprobs[i] if batch.logprobs else None
            if lp is not None:  # add the text of every token so clients need no tokenizer
                lp = dict(lp, tokens=[self.tokenizer.decode([t]) for t in ids[: len(lp["token_logprobs"])]],
                          top_tokens=[[self.tokenizer.decode([t]) for t, _ in row] for row in lp["top_logprobs"]])
            out.logprobs.append(lp)
        return out


def run_detokenizer_process(tokenizer_path, recv_addr, send_addr: str, pipe_writer=None, vocab_size: int = 1024,
                            tokenizer_mode: str = "auto", trust_remote_code: bool = False, log_level: str = "info") -> None:
    import zmq

    from .ipc_utils import make_socket, setup_subprocess_logging

    setup_subprocess_logging(log_level)
    worker = DetokenizerWorker(tokenizer_path, vocab_size, tokenizer_mode, trust_remote_code)
    ctx = zmq.Context()
    # one endpoint per engine replica (data parallelism): a PULL socket fair-queues over all of them
    addrs = [recv_addr] if isinstance(recv_addr, str) else list(recv_addr)
    recv = make_socket(ctx, zmq.PULL, addrs[0], bind=False)
    for a in addrs[1:]:
        recv.connect(a)
    send = make_socket(ctx, zmq.PUSH, send_addr, bind=True)
    if pipe_writer is not None:
        pipe_writer.send({"status": "ready"})
    open_replicas = len(addrs)
    while True:
        msg = recv.recv_pyobj()
        if msg is None:  # a replica's scheduler has shut down
            open_replicas -= 1
            if open_replicas <= 0:
                return
            continue
        if isinstance(msg, BatchTokenIDOutput):
            send.send_pyobj(worker.detokenize(msg))
        else:
            send.send_pyobj(msg)  # errors and control replies pass through

"""Tokenizer worker (role of pymllm/orchestrator/tokenizer_process.py:44-523): text -> ids with
truncation to the context length; images (path / bytes / PIL / arrays) go through the model's
processor when one exists, whose ``input_ids`` then replace the text ids; forwards
``TokenizedGenerateReqInput`` to the scheduler and passes aborts through.  In a data-parallel
deployment (several engine replicas) the worker is also the router that spreads the requests."""

from __future__ import annotations

import hashlib
import io
import logging
import time
from collections import OrderedDict
from typing import Any, Dict, List, Optional, Sequence, Union

from ..engine.io_struct import AbortReq, FlushCacheReq, SharedQueueNotice, TokenizedGenerateReqInput
from ..utils.tokenizer import get_tokenizer

logger = logging.getLogger(__name__)


class TokenizerWorker:
    def __init__(self, tokenizer_path, context_length: Optional[int] = None, vocab_size: int = 1024,
                 tokenizer_mode: str = "auto", trust_remote_code: bool = False, mm_config: Optional[Dict[str, Any]] = None) -> None:
        self.tokenizer = get_tokenizer(tokenizer_path, vocab_size, tokenizer_mode, trust_remote_code)
        self.context_length = context_length
        self.processor = self._load_processor(tokenizer_path, trust_remote_code)
        # ids and patch geometry of the model's vision tokens: lets images be served without a HF
        # processor (random-init presets, checkpoints shipped without preprocessor_config.json)
        self.mm_config = mm_config

    @staticmethod
    def _load_processor(path, trust_remote_code):
        import os

        s = str(path) if path is not None else ""
        if not s or s.startswith("preset:") or not os.path.exists(os.path.join(s, "preprocessor_config.json")):
            return None
        try:
            from transformers import AutoProcessor

            return AutoProcessor.from_pretrained(s, trust_remote_code=trust_remote_code)
        except Exception as exc:  # text-only serving still works
            logger.warning("no multimodal processor: %s", exc)
            return None

    @staticmethod
    def load_image(item: Any):
        """path / URL-less data URI / bytes / PIL image / array -> PIL image."""
        from PIL import Image

        if isinstance(item, Image.Image):
            return item.convert("RGB")
        if isinstance(item, (bytes, bytearray)):
            return Image.open(io.BytesIO(item)).convert("RGB")
        if isinstance(item, str):
            if item.startswith("data:"):
                import base64

                return Image.open(io.BytesIO(base64.b64decode(item.split(",", 1)[1]))).convert("RGB")
            return Image.open(item).convert("RGB")
        import numpy as np

        return Image.fromarray(np.asarray(item).astype("uint8")).convert("RGB")

    def _builtin_image_inputs(self, images, text, ids):
        """Built-in preprocessing: every image becomes ``<vision_start> <image_pad> * n <vision_end>`` in
        front of the text tokens; pixels are patchified by :mod:`mllm_b200.utils.image_processor`."""
        import numpy as np
        import torch

        from ..utils.image_processor import image_token_count, preprocess_image

        mc = self.mm_config
        text_ids = list(ids) if ids is not None else self.tokenizer.encode(text or "")
        pix, grids, block, h = [], [], [], hashlib.sha256()
        for item in (images if isinstance(images, list) else [images]):
            arr = item if isinstance(item, (np.ndarray, torch.Tensor)) else np.asarray(self.load_image(item))
            img = torch.as_tensor(np.asarray(arr)).to(torch.uint8)
            h.update(img.numpy().tobytes())
            pv, g = preprocess_image(img, mc["patch_size"], mc["merge_size"], mc["temporal_patch_size"],
                                     mean=mc.get("image_mean", 0.5), std=mc.get("image_std", 0.5))
            pix.append(pv)
            grids.append(g)
            block += [mc["vision_start_token_id"]] + [mc["image_token_id"]] * image_token_count(g, mc["merge_size"]) + \
                [mc["vision_end_token_id"]]
        mm = {"pixel_values": torch.cat(pix), "image_grid_thw": torch.cat(grids), "image_hash": h.hexdigest()[:16]}
        return block + text_ids, mm

    def tokenize(self, req: Dict[str, Any]) -> TokenizedGenerateReqInput:
        text = req.get("text")
        ids = req.get("input_ids")
        mm_inputs = None
        images = req.get("image_data")
        if images is not None and self.processor is not None:
            imgs = [self.load_image(i) for i in (images if isinstance(images, list) else [images])]
            out = self.processor(images=imgs, text=text or "", return_tensors="pt")
            ids = out["input_ids"][0].tolist()
            h = hashlib.sha256()
            for im in imgs:
                h.update(im.tobytes())
            mm_inputs = {"pixel_values": out.get("pixel_values"), "image_grid_thw": out.get("image_grid_thw"),
                         "image_hash": h.hexdigest()[:16]}
        elif images is not None and self.mm_config is not None:
            ids, mm_inputs = self._builtin_image_inputs(images, text, ids)
        elif ids is None:
            ids = self.tokenizer.encode(text or "")
        ids = list(ids)
        if self.context_length and len(ids) >= self.context_length:
            ids = ids[: self.context_length - 1]
        return TokenizedGenerateReqInput(
            rid=req["rid"], input_text=text or "", input_ids=ids, mm_inputs=mm_inputs,
            sampling_params=req.get("sampling_params") or {}, stream=bool(req.get("stream", False)),
            return_logprob=bool(req.get("return_logprob") or False), top_logprobs_num=int(req.get("top_logprobs_num") or 0),
            created_time=req.get("created_time") or time.time())


class ReplicaRouter:
    """Hands tokenised requests to the engine replicas of a data-parallel deployment.

    Every replica is a complete scheduler + model runner (group) with its own KV pool and prefix
    cache.  Requests go to the replica with the fewest prompt tokens assigned so far among those
    dispatched in the current window (ties: round robin), which keeps long and short prompts spread
    evenly without feedback from the schedulers; an abort follows its request; cache flushes and the
    shutdown marker go to every replica."""

    WINDOW = 64        # requests after which the per-replica token tallies start again
    MAX_TRACKED = 1 << 16

    def __init__(self, senders: Sequence[Any], shared_queues: Optional[Sequence[Any]] = None) -> None:
        self.senders = list(senders)
        # one shared-memory queue per replica: requests that carry tensors (images) take it, the socket
        # then only carries a notice
        self.shared_queues = list(shared_queues) if shared_queues else None
        self.load = [0] * len(self.senders)
        self.count = 0
        self.next = 0
        self.owner: "OrderedDict[str, int]" = OrderedDict()

    def pick(self, tokens: int) -> int:
        n = len(self.senders)
        if self.count % self.WINDOW == 0:
            self.load = [0] * n
        self.count += 1
        order = [(self.next + i) % n for i in range(n)]
        best = min(order, key=lambda r: self.load[r])
        self.load[best] += max(1, tokens)
        self.next = (best + 1) % n
        return best

    def route(self, msg: Any) -> List[int]:
        """Sends ``msg`` and returns the replica indices it went to."""
        n = len(self.senders)
        if msg is None or isinstance(msg, FlushCacheReq):
            targets = list(range(n))
        elif isinstance(msg, AbortReq):
            r = self.owner.pop(msg.rid, None)
            targets = [r] if r is not None else list(range(n))
        else:
            r = self.pick(len(getattr(msg, "input_ids", None) or ()))
            self.owner[msg.rid] = r
            while len(self.owner) > self.MAX_TRACKED:
                self.owner.popitem(last=False)
            targets = [r]
        for r in targets:
            if (self.shared_queues is not None and isinstance(msg, TokenizedGenerateReqInput)
                    and msg.mm_inputs is not None):
                import dataclasses

                self.shared_queues[r].put(msg.rid, dataclasses.replace(msg, mm_inputs=None), msg.mm_inputs)
                self.senders[r].send_pyobj(SharedQueueNotice(rid=msg.rid))
            else:
                self.senders[r].send_pyobj(msg)
        return targets


def run_tokenizer_process(tokenizer_path, recv_addr: str, send_addr: Union[str, Sequence[str]], pipe_writer=None,
                          context_length: Optional[int] = None, vocab_size: int = 1024, tokenizer_mode: str = "auto",
                          trust_remote_code: bool = False, log_level: str = "info",
                          mm_config: Optional[Dict[str, Any]] = None, shared_queues: Optional[Sequence[Any]] = None) -> None:
    """``send_addr``: one endpoint, or one per data-parallel replica; ``shared_queues``: the matching
    ``TensorQueue`` objects when the shared-memory fast path is on."""
    import zmq

    from .ipc_utils import make_socket, setup_subprocess_logging

    setup_subprocess_logging(log_level)
    worker = TokenizerWorker(tokenizer_path, context_length, vocab_size, tokenizer_mode, trust_remote_code, mm_config)
    ctx = zmq.Context()
    recv = make_socket(ctx, zmq.PULL, recv_addr, bind=False)
    addrs = [send_addr] if isinstance(send_addr, str) else list(send_addr)
    router = ReplicaRouter([make_socket(ctx, zmq.PUSH, a, bind=True) for a in addrs], shared_queues)
    if pipe_writer is not None:
        pipe_writer.send({"status": "ready"})
    while True:
        msg = recv.recv_pyobj()
        if msg is None:
            router.route(None)
            return
        if isinstance(msg, (AbortReq, FlushCacheReq)):
            router.route(msg)
            continue
        try:
            router.route(worker.tokenize(msg))
        except Exception as exc:
            logger.exception("tokenization failed")
            router.route(AbortReq(rid=msg.get("rid", "")))

"""Tokenizer worker (role of pymllm/orchestrator/tokenizer_process.py:44-523): text -> ids with
truncation to the context length; images (path / bytes / PIL / arrays) go through the model's
processor when one exists, whose ``input_ids`` then replace the text ids; forwards
``TokenizedGenerateReqInput`` to the scheduler and passes aborts through.  In a data-parallel
deployment (several engine replicas) the worker is also the router that spreads the requests."""

from __future__ import annotations

import hashlib
import io
import logging
import os
import time
from collections import OrderedDict
from typing import Any, Dict, List, Optional, Sequence, Union

from ..engine.io_struct import AbortReq, FlushCacheReq, SharedQueueNotice, TokenizedGenerateReqInput
from ..utils.tokenizer import get_tokenizer

logger = logging.getLogger(__name__)


def _is_frame_list(v) -> bool:
    """A list whose entries are single frames (one video given as its frames), not a list of videos."""
    import numpy as np

    if not isinstance(v, (list, tuple)) or not v:
        return False
    first = v[0]
    if isinstance(first, (dict, list, tuple)):
        return False
    if isinstance(first, str):      # image files are frames; array files, containers and video data URIs are whole videos
        return not (first.endswith(".npy") or first.startswith("data:video/")
                    or first.lower().endswith(TokenizerWorker._CONTAINER_EXT))
    return not (hasattr(first, "ndim") and np.ndim(first) == 4)


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

    # remote media: fetched with a time limit and a size cap; MLLM_B200_FETCH_URLS=0 refuses every remote URL
    _FETCH_TIMEOUT_S = 10.0
    _FETCH_MAX_BYTES = 256 << 20

    @classmethod
    def fetch_url(cls, url: str) -> bytes:
        """The bytes behind an ``http(s)://`` URL of an image or video part."""
        if os.environ.get("MLLM_B200_FETCH_URLS", "1") == "0":
            raise ValueError("remote media URLs are disabled on this server (MLLM_B200_FETCH_URLS=0): send the data inline")
        import urllib.request

        try:
            with urllib.request.urlopen(url, timeout=cls._FETCH_TIMEOUT_S) as r:
                data = r.read(cls._FETCH_MAX_BYTES + 1)
        except Exception as e:
            raise ValueError(f"could not fetch {url!r}: {type(e).__name__}: {e}") from e
        if len(data) > cls._FETCH_MAX_BYTES:
            raise ValueError(f"{url!r} is larger than {cls._FETCH_MAX_BYTES >> 20} MiB")
        return data

    @classmethod
    def load_image(cls, item: Any):
        """path / http(s) URL / data URI / bytes / PIL image / array -> PIL image."""
        from PIL import Image

        if isinstance(item, Image.Image):
            return item.convert("RGB")
        if isinstance(item, (bytes, bytearray)):
            return Image.open(io.BytesIO(item)).convert("RGB")
        if isinstance(item, str):
            if item.startswith("data:"):
                import base64

                return Image.open(io.BytesIO(base64.b64decode(item.split(",", 1)[1]))).convert("RGB")
            if item.startswith(("http://", "https://")):
                return Image.open(io.BytesIO(cls.fetch_url(item))).convert("RGB")
            if item.startswith("file://"):
                item = item[len("file://"):]
            return Image.open(item).convert("RGB")
        import numpy as np

        return Image.fromarray(np.asarray(item).astype("uint8")).convert("RGB")

    @classmethod
    def load_video(cls, item: Any):
        """-> (uint8 frames ``[F, H, W, 3]`` as a tensor, frames per second of that frame list or None).

        Accepted: an array / tensor ``[F, H, W, 3]``; a list of frames (anything :meth:`load_image` takes, or
        arrays); a ``.npy`` file holding such an array; a container file (mp4, avi, mov, mkv, webm, ...: decoded with
        OpenCV when it is installed), its bytes or a ``data:video/...;base64,`` URI; a dict
        ``{"frames": <any of these>, "fps": f}`` (``f`` overrides the container's own rate)."""
        import numpy as np
        import torch

        src = cls._container_source(item)
        if src is not None:
            path, fps, cleanup = src
            try:
                total, own_fps = cls._probe_container(path)
                return cls._decode_container(path, None), float(fps or own_fps or 0.0) or None
            finally:
                cleanup()
        fps = None
        if isinstance(item, dict):
            fps = item.get("fps")
            item = item.get("frames")
        if isinstance(item, str):
            if not item.endswith(".npy"):
                raise ValueError(f"video_data: {item!r} is neither a .npy file nor a video container this build can open")
            item = np.load(item)
        if isinstance(item, (list, tuple)):
            frames = [np.asarray(f) if isinstance(f, (np.ndarray, torch.Tensor)) else np.asarray(cls.load_image(f)) for f in item]
            if not frames or any(f.shape != frames[0].shape for f in frames):
                raise ValueError("video_data: frames must be non-empty and share one size")
            item = np.stack(frames)
        arr = torch.as_tensor(np.asarray(item))
        if arr.dim() != 4 or arr.shape[-1] != 3:
            raise ValueError(f"video_data: expected frames [F, H, W, 3], got {tuple(arr.shape)}")
        return arr.to(torch.uint8), (float(fps) if fps else None)

    # ---- container files (mp4, ...) through OpenCV's FFmpeg reader ----
    _CONTAINER_EXT = (".mp4", ".m4v", ".mov", ".avi", ".mkv", ".webm", ".mpg", ".mpeg", ".wmv", ".flv", ".gif")

    @classmethod
    def _container_source(cls, item: Any):
        """``(path, fps override, cleanup)`` when ``item`` names or holds a container file, else None.  Bytes and
        data URIs are written to a temporary file (the reader wants a path); ``cleanup()`` removes it."""
        fps = None
        if isinstance(item, dict):
            fps = item.get("fps")
            item = item.get("frames", item.get("path"))
        nothing = lambda: None  # noqa: E731
        if isinstance(item, os.PathLike):
            item = os.fspath(item)
        if isinstance(item, str) and item.startswith("file://"):
            item = item[len("file://"):]
        if isinstance(item, str) and item.startswith(("http://", "https://")):
            item = cls.fetch_url(item)
        if isinstance(item, str) and item.lower().endswith(cls._CONTAINER_EXT):
            return item, fps, nothing
        data = None
        if isinstance(item, str) and item.startswith("data:video/"):
            import base64

            data = base64.b64decode(item.split(",", 1)[1])
        elif isinstance(item, (bytes, bytearray)):
            data = bytes(item)
        if data is None:
            return None
        import tempfile

        f = tempfile.NamedTemporaryFile(suffix=".mp4", delete=False)
        f.write(data)
        f.close()
        return f.name, fps, lambda: os.path.exists(f.name) and os.unlink(f.name)

    @staticmethod
    def _cv2():
        try:
            import cv2
        except ImportError as e:
            raise ValueError("video_data: container formats need OpenCV (cv2) to be decoded; pass frames instead") from e
        return cv2

    @classmethod
    def _probe_container(cls, path: str):
        """(frame count the container declares, its frames per second)."""
        cv2 = cls._cv2()
        cap = cv2.VideoCapture(path)
        try:
            if not cap.isOpened():
                raise ValueError(f"video_data: cannot open {path!r} as a video")
            return int(cap.get(cv2.CAP_PROP_FRAME_COUNT) or 0), float(cap.get(cv2.CAP_PROP_FPS) or 0.0)
        finally:
            cap.release()

    @classmethod
    def _decode_container(cls, path: str, keep: Optional[Sequence[int]]):
        """uint8 RGB frames ``[F, H, W, 3]``: all of them, or the frame numbers ``keep`` (ascending; frames in
        between are skipped without being converted).  A file that ends before its declared length gives fewer."""
        import numpy as np
        import torch

        cv2 = cls._cv2()
        cap = cv2.VideoCapture(path)
        if not cap.isOpened():
            raise ValueError(f"video_data: cannot open {path!r} as a video")
        want = None if keep is None else list(keep)
        out, i, k = [], 0, 0
        try:
            while want is None or k < len(want):
                if not cap.grab():
                    break
                while want is not None and k < len(want) and want[k] < i:
                    k += 1                                   # repeated or unsorted entries: take what still lies ahead
                if want is None or (k < len(want) and want[k] == i):
                    ok, frame = cap.retrieve()
                    if not ok:
                        break
                    rgb = np.ascontiguousarray(frame[..., ::-1])
                    reps = 1
                    if want is not None:
                        reps = 0
                        while k < len(want) and want[k] == i:
                            reps, k = reps + 1, k + 1
                    out.extend([rgb] * reps)
                i += 1
        finally:
            cap.release()
        if not out:
            raise ValueError(f"video_data: no frame could be decoded from {path!r}")
        return torch.from_numpy(np.stack(out)).to(torch.uint8)

    @classmethod
    def load_video_sampled(cls, item: Any, sampler):
        """``(kept frames, their frame numbers, frames per second of the source, frame count of the source)``;
        ``sampler(total, fps)`` picks the frame numbers.  A container is decoded only at those frames."""
        src = cls._container_source(item)
        if src is None:
            frames, fps = cls.load_video(item)
            src_fps = fps or 24.0
            keep = list(sampler(int(frames.shape[0]), src_fps))
            return frames[keep], keep, src_fps, int(frames.shape[0])
        path, fps, cleanup = src
        try:
            total, own_fps = cls._probe_container(path)
            src_fps = float(fps or own_fps or 24.0)
            if total <= 0:                                   # no declared length: decode, then sample
                frames = cls._decode_container(path, None)
                keep = list(sampler(int(frames.shape[0]), src_fps))
                return frames[keep], keep, src_fps, int(frames.shape[0])
            keep = list(sampler(total, src_fps))
            frames = cls._decode_container(path, keep)
            return frames, keep[: int(frames.shape[0])], src_fps, total
        finally:
            cleanup()

    def _builtin_mm_inputs(self, images, videos, text, ids):
        """Built-in preprocessing.  Every image becomes ``<vision_start> <image_pad> * n <vision_end>``.  A video
        depends on the family (``video_layout``): ``"frames"`` writes ``"<t seconds>" <vision_start> <video_pad> * n
        <vision_end>`` per temporal patch (the layout of the Qwen3-VL processor), each stored like an image of grid
        ``[1, h, w]``; ``"clip"`` writes one ``<vision_start> <video_pad> * (T n) <vision_end>`` block of grid
        ``[T, h, w]`` (Qwen2-VL, Qwen2.5-VL), and with ``tokens_per_second`` set the temporal position advances by
        ``seconds per temporal patch x tokens_per_second`` per patch (``mrope_t_scale``).  The blocks go in front of
        the text tokens unless the text holds placeholders.  Pixels are patchified by
        :mod:`mllm_b200.utils.image_processor`; the model sees one list of grids in order of appearance."""
        import numpy as np
        import torch

        from ..utils.image_processor import (image_token_count, preprocess_image, preprocess_video, sample_frame_indices,
                                             sample_frame_indices_strided, video_timestamps)

        mc = self.mm_config
        text_ids = list(ids) if ids is not None else self.tokenizer.encode(text or "")
        pix, grids, h = [], [], hashlib.sha256()
        blocks = []                     # (kind token, token ids of the block, pixel rows, grid rows, temporal step)
        norm = dict(mean=mc.get("image_mean", 0.5), std=mc.get("image_std", 0.5))
        for item in ([] if images is None else images if isinstance(images, list) else [images]):
            arr = item if isinstance(item, (np.ndarray, torch.Tensor)) else np.asarray(self.load_image(item))
            img = torch.as_tensor(np.array(arr)).to(torch.uint8)
            h.update(img.numpy().tobytes())
            pv, g = preprocess_image(img, mc["patch_size"], mc["merge_size"], mc["temporal_patch_size"], **norm)
            blocks.append((mc["image_token_id"], [mc["vision_start_token_id"]] + [mc["image_token_id"]] *
                           image_token_count(g, mc["merge_size"]) + [mc["vision_end_token_id"]], pv, g, [1.0]))
        if videos is not None and mc.get("video_token_id") is None:
            raise ValueError("this model has no video token: video_data is not supported")
        for item in ([] if videos is None else videos if isinstance(videos, list) and not _is_frame_list(videos) else [videos]):
            target, lo, hi = float(mc.get("video_fps", 2.0)), int(mc.get("video_min_frames", 4)), int(mc.get("video_max_frames", 768))
            if mc.get("video_layout", "frames") == "clip":
                frames, keep, src_fps, total = self.load_video_sampled(
                    item, lambda n, f: sample_frame_indices_strided(n, f, target, lo, hi, mc["temporal_patch_size"]))
                h.update(frames.numpy().tobytes())
                unit = (mc["patch_size"] * mc["merge_size"]) ** 2
                pv, g = preprocess_video(frames, mc["patch_size"], mc["merge_size"], mc["temporal_patch_size"],
                                         min_pixels=128 * unit, max_pixels=768 * unit, **norm)
                T, gh, gw = (int(v) for v in g[0])
                per = (gh // mc["merge_size"]) * (gw // mc["merge_size"])
                block = [mc["vision_start_token_id"]] + [mc["video_token_id"]] * (T * per) + [mc["vision_end_token_id"]]
                step = 1.0
                if mc.get("tokens_per_second"):
                    sampled_fps = len(keep) / max(total, 1) * src_fps
                    step = mc["temporal_patch_size"] / max(sampled_fps, 1e-6) * float(mc["tokens_per_second"])
                blocks.append((mc["video_token_id"], block, pv, g, [step]))
                continue
            frames, keep, src_fps, _ = self.load_video_sampled(item, lambda n, f: sample_frame_indices(n, f, target, lo, hi))
            h.update(frames.numpy().tobytes())
            pv, g = preprocess_video(frames, mc["patch_size"], mc["merge_size"], mc["temporal_patch_size"], **norm)
            T, gh, gw = (int(v) for v in g[0])
            per = (gh // mc["merge_size"]) * (gw // mc["merge_size"])
            block = []
            for t in video_timestamps(keep, src_fps, mc["temporal_patch_size"]):
                block += self.tokenizer.encode(f"<{t:.1f} seconds>") + [mc["vision_start_token_id"]] + \
                    [mc["video_token_id"]] * per + [mc["vision_end_token_id"]]
            blocks.append((mc["video_token_id"], block, pv, torch.tensor([[1, gh, gw]] * T, dtype=torch.int64), [1.0] * T))
        # a block replaces its placeholder  <vision_start> <pad> <vision_end>  in the text (chat templates write
        # one per image / video part), in order of appearance; blocks without one go in front of the text
        vs, ve = mc["vision_start_token_id"], mc["vision_end_token_id"]
        out_ids, placed, i = [], [False] * len(blocks), 0
        body = []                                     # (ids chunk, block index or None) in text order
        while i < len(text_ids):
            if text_ids[i] == vs and i + 2 < len(text_ids) and text_ids[i + 2] == ve:
                j = next((b for b, blk in enumerate(blocks) if not placed[b] and blk[0] == text_ids[i + 1]), None)
                if j is not None:
                    placed[j] = True
                    body.append((blocks[j][1], j))
                    i += 3
                    continue
            body.append(([text_ids[i]], None))
            i += 1
        order = [b for b in range(len(blocks)) if not placed[b]] + [j for _, j in body if j is not None]
        for b in range(len(blocks)):
            if not placed[b]:
                out_ids += blocks[b][1]
        for chunk, _ in body:
            out_ids += chunk
        steps = []
        for b in order:
            pix.append(blocks[b][2])
            grids.append(blocks[b][3])
            steps += blocks[b][4]
        mm = {"pixel_values": torch.cat(pix), "image_grid_thw": torch.cat(grids), "image_hash": h.hexdigest()[:16]}
        if any(v != 1.0 for v in steps):
            mm["mrope_t_scale"] = torch.tensor(steps, dtype=torch.float64)
        return out_ids, mm

    @staticmethod
    def merge_vision_inputs(ids, image_pixels, image_grids, video_pixels, video_grids, image_token_id: int,
                            video_token_id: int, vision_start_token_id: int, merge_size: int, video_steps=None):
        """One ``(pixel_values, grid_thw)`` list in order of appearance from a processor's separate image and
        video outputs.  Walks the vision-start tokens of ``ids``: an image block takes the next image grid; a
        video block takes the next temporal patch of the current video as grid ``[1, h, w]`` (a video of grid
        ``[T, h, w]`` whose prompt has one block per temporal patch), or the whole ``[T, h, w]`` grid when the
        block holds all of its tokens.  With ``video_steps`` (one temporal position step per video) a third value
        is returned: the step of every merged grid, 1 for images."""
        import torch

        ig = [] if image_grids is None else image_grids.tolist()
        vg = [] if video_grids is None else video_grids.tolist()
        pix, grids, steps = [], [], []
        i_img = i_vid = t_in_vid = 0
        img_row = vid_row = 0
        n = len(ids)
        for k, tok in enumerate(ids):
            if tok != vision_start_token_id or k + 1 >= n:
                continue
            if ids[k + 1] == image_token_id and i_img < len(ig):
                t, hh, ww = ig[i_img]
                rows = t * hh * ww
                pix.append(image_pixels[img_row:img_row + rows])
                grids.append([t, hh, ww])
                steps.append(1.0)
                img_row += rows
                i_img += 1
            elif ids[k + 1] == video_token_id and i_vid < len(vg):
                t, hh, ww = vg[i_vid]
                per = (hh // merge_size) * (ww // merge_size)
                run = 0
                while k + 1 + run < n and ids[k + 1 + run] == video_token_id:
                    run += 1
                if run >= t * per and t_in_vid == 0:          # the whole video in one block
                    take = t
                else:
                    take = 1
                rows = take * hh * ww
                pix.append(video_pixels[vid_row:vid_row + rows])
                grids.append([take, hh, ww])
                steps.append(float(video_steps[i_vid]) if video_steps is not None else 1.0)
                vid_row += rows
                t_in_vid += take
                if t_in_vid >= t:
                    i_vid, t_in_vid = i_vid + 1, 0
        if not pix:
            return (None, None) if video_steps is None else (None, None, None)
        out = torch.cat(pix), torch.tensor(grids, dtype=torch.int64)
        return out if video_steps is None else out + (torch.tensor(steps, dtype=torch.float64),)

    def _processor_mm_inputs(self, images, videos, text):
        """Through the checkpoint's own HF processor; its separate image / video outputs are merged into one list
        in order of appearance (:meth:`merge_vision_inputs`)."""
        h = hashlib.sha256()
        kw = {}
        if images is not None:
            kw["images"] = [self.load_image(i) for i in (images if isinstance(images, list) else [images])]
            for im in kw["images"]:
                h.update(im.tobytes())
        if videos is not None:
            vids = videos if isinstance(videos, list) and not _is_frame_list(videos) else [videos]
            loaded = [self.load_video(v) for v in vids]
            kw["videos"] = [f.numpy() for f, _ in loaded]
            for f, _ in loaded:
                h.update(f.numpy().tobytes())
            fps = [fp for _, fp in loaded]
            if all(fp is not None for fp in fps):
                kw["video_metadata"] = [dict(fps=fp, total_num_frames=int(f.shape[0]), frames_indices=list(range(int(f.shape[0]))))
                                        for (f, _), fp in zip(loaded, fps)]
                kw["do_sample_frames"] = False
        out = self.processor(text=text or "", return_tensors="pt", **kw)
        ids = out["input_ids"][0].tolist()
        pv, grid = out.get("pixel_values"), out.get("image_grid_thw")
        steps = None
        if out.get("pixel_values_videos") is not None:
            mc = self.mm_config or {}
            tok = self.processor
            if mc.get("tokens_per_second") and out.get("second_per_grid_ts") is not None:
                steps = [float(v) * float(mc["tokens_per_second"]) for v in out["second_per_grid_ts"]]
            merged = self.merge_vision_inputs(
                ids, pv, grid, out["pixel_values_videos"], out["video_grid_thw"],
                int(mc.get("image_token_id", getattr(tok, "image_token_id", -1))),
                int(mc.get("video_token_id", getattr(tok, "video_token_id", -1))),
                int(mc.get("vision_start_token_id", getattr(tok, "vision_start_token_id", -1))),
                int(mc.get("merge_size", 2)), video_steps=steps)
            pv, grid = merged[0], merged[1]
            steps = merged[2] if steps is not None else None
        mm = {"pixel_values": pv, "image_grid_thw": grid, "image_hash": h.hexdigest()[:16]}
        if steps is not None and bool((steps != 1.0).any()):
            mm["mrope_t_scale"] = steps
        return ids, mm

    def tokenize(self, req: Dict[str, Any]) -> TokenizedGenerateReqInput:
        text = req.get("text")
        ids = req.get("input_ids")
        mm_inputs = None
        images, videos = req.get("image_data"), req.get("video_data")
        if (images is not None or videos is not None) and self.processor is not None:
            ids, mm_inputs = self._processor_mm_inputs(images, videos, text)
        elif (images is not None or videos is not None) and self.mm_config is not None:
            ids, mm_inputs = self._builtin_mm_inputs(images, videos, text, ids)
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

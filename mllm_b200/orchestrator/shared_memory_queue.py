"""Tokenizer -> scheduler hand-off of multimodal requests: a POSIX shared-memory lane for the pickled
metadata (read once, unlinked by the reader) and a queue lane for tensors (roles of
pymllm/orchestrator/shared_memory_queue.py:67-292).

Three transport modes for the tensors inside ``mm_inputs``:

* ``"default"``       — tensors stay on the host and travel through the queue (shared CPU memory);
* ``"cuda_ipc"``      — device tensors travel as CUDA IPC handles (the receiver maps the sender's
  allocation; the sender keeps it alive until the receiver confirms);
* ``"cuda_ipc_pool"`` — device tensors are first copied into a fixed device workspace
  (``MmItemMemoryPool``) whose chunks are recycled when the receiver flips a shared flag, so no
  allocation is ever exported twice and the sender never blocks on the receiver.
"""

from __future__ import annotations

import logging
import multiprocessing as mp
import pickle
import uuid
from multiprocessing.shared_memory import SharedMemory
from typing import Any, Optional, Tuple

import torch

from .cuda_ipc_transport import MmItemMemoryPool, unwrap_mm_inputs, wrap_mm_inputs

logger = logging.getLogger(__name__)
TRANSPORT_MODES = ("default", "cuda_ipc", "cuda_ipc_pool")


class SharedMemoryManager:
    """One shared-memory segment per request's metadata; the reader unlinks it."""

    PREFIX = "mllm_b200_meta_"

    @staticmethod
    def write_metadata(rid: str, metadata: Any) -> str:
        data = pickle.dumps(metadata, protocol=pickle.HIGHEST_PROTOCOL)
        name = f"{SharedMemoryManager.PREFIX}{rid}_{uuid.uuid4().hex[:8]}"
        shm = SharedMemory(name=name, create=True, size=max(1, len(data) + 8))
        shm.buf[:8] = len(data).to_bytes(8, "little")  # segments are page-rounded: keep the true length
        shm.buf[8:8 + len(data)] = data
        shm.close()
        return name

    @staticmethod
    def read_metadata(shm_name: str, unlink: bool = True) -> Any:
        shm = SharedMemory(name=shm_name, create=False)
        try:
            n = int.from_bytes(bytes(shm.buf[:8]), "little")
            return pickle.loads(bytes(shm.buf[8:8 + n]))
        finally:
            shm.close()
            if unlink:
                try:
                    shm.unlink()
                except FileNotFoundError:
                    pass

    @staticmethod
    def cleanup(shm_name: str) -> None:
        try:
            shm = SharedMemory(name=shm_name, create=False)
            shm.close()
            shm.unlink()
        except FileNotFoundError:
            pass


class TensorQueue:
    """``put(rid, metadata, mm_inputs)`` / ``get()`` across processes."""

    def __init__(self, maxsize: int = 0, transport_mode: str = "default", pool: Optional[MmItemMemoryPool] = None,
                 ctx: Optional[mp.context.BaseContext] = None) -> None:
        if transport_mode not in TRANSPORT_MODES:
            raise ValueError(f"transport_mode must be one of {TRANSPORT_MODES}")
        self.mode = transport_mode
        self.pool = pool
        self._q = (ctx or mp.get_context("spawn")).Queue(maxsize)

    def put(self, rid: str, metadata: Any, mm_inputs: Any = None, block: bool = True, timeout: Optional[float] = None) -> None:
        name = SharedMemoryManager.write_metadata(rid, metadata)
        try:
            payload = self._outgoing(mm_inputs)
            self._q.put((rid, name, payload), block=block, timeout=timeout)
        except Exception:
            SharedMemoryManager.cleanup(name)
            raise

    def get(self, block: bool = True, timeout: Optional[float] = None) -> Tuple[str, Any, Any]:
        rid, name, payload = self._q.get(block=block, timeout=timeout)
        return rid, SharedMemoryManager.read_metadata(name), unwrap_mm_inputs(payload)

    def _outgoing(self, data: Any) -> Any:
        if data is None:
            return None
        if self.mode == "default":
            return _to_shared_cpu(data)
        return wrap_mm_inputs(data, pool=self.pool if self.mode == "cuda_ipc_pool" else None)

    def empty(self) -> bool:
        return self._q.empty()

    def qsize(self) -> int:
        try:
            return self._q.qsize()
        except NotImplementedError:  # macOS
            return 0

    def close(self) -> None:
        self._q.close()
        if self.pool is not None:
            self.pool.shutdown()


def _to_shared_cpu(data: Any) -> Any:
    if isinstance(data, torch.Tensor):
        t = data.detach().cpu()
        return t.share_memory_() if t.numel() else t
    if isinstance(data, dict):
        return {k: _to_shared_cpu(v) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(_to_shared_cpu(v) for v in data)
    return data

"""Device tensors across processes without a host copy (roles of
pymllm/orchestrator/cuda_ipc_transport.py:75-648).

``CudaIpcTensorTransportProxy`` pickles as a CUDA IPC handle of the tensor's allocation plus shape,
dtype, stride and offset; ``reconstruct_on_device`` maps it in the receiver, copies into receiver-owned
memory (so the sender's buffer can be reused) and flips the shared sync flag.  ``MmItemMemoryPool``
is the sender-side fixed workspace: multimodal tensors are copied into chunks of one device buffer,
each chunk guarded by a one-int shared-memory flag that the receiver sets when it is done; a recycler
thread returns flagged chunks and merges neighbours.  Host tensors pass through untouched.
"""

from __future__ import annotations

import logging
import threading
import time
import uuid
from multiprocessing.shared_memory import SharedMemory
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

logger = logging.getLogger(__name__)


class ShmSyncBuffer:
    """One int32 in POSIX shared memory: number of consumers that have finished with a chunk."""

    def __init__(self, name: Optional[str] = None, create: bool = True) -> None:
        self.name = name or f"mllm_b200_sync_{uuid.uuid4().hex[:12]}"
        self._shm = SharedMemory(name=self.name, create=create, size=4)
        self._arr = np.ndarray((1,), dtype=np.int32, buffer=self._shm.buf)
        self._owner = create
        if create:
            self._arr[0] = 0

    @classmethod
    def open(cls, name: str) -> "ShmSyncBuffer":
        return cls(name=name, create=False)

    @property
    def value(self) -> int:
        return int(self._arr[0])

    def reset(self) -> None:
        self._arr[0] = 0

    def signal(self) -> None:
        self._arr[0] += 1  # one consumer per chunk in this runtime (the scheduler / model-runner rank)

    def close(self) -> None:
        self._arr = None
        try:
            self._shm.close()
            if self._owner:
                self._shm.unlink()
        except (FileNotFoundError, BufferError):
            pass


class MmItemMemoryChunk:
    def __init__(self, area: Tuple[int, int], sync_flag: ShmSyncBuffer) -> None:
        self.area = area            # [start, end) in bytes inside the workspace
        self.sync_flag = sync_flag

    @property
    def start(self) -> int:
        return self.area[0]

    @property
    def end(self) -> int:
        return self.area[1]

    @property
    def mem_size(self) -> int:
        return self.area[1] - self.area[0]

    def try_to_recycle(self, num_consumers: int = 1) -> bool:
        if self.sync_flag.value >= num_consumers:
            self.sync_flag.reset()
            return True
        return False


class MmItemMemoryPool:
    """Fixed byte workspace on ``device`` carved into chunks (first fit, 256-byte aligned)."""

    ALIGN = 256

    def __init__(self, size_bytes: int, device: torch.device | str = "cuda", num_consumers: int = 1,
                 recycle_interval_s: float = 0.05, start_recycler: bool = True) -> None:
        self.device = torch.device(device)
        self.size = int(size_bytes) // self.ALIGN * self.ALIGN
        self.workspace = torch.empty(self.size, dtype=torch.uint8, device=self.device)
        self.num_consumers = num_consumers
        self._lock = threading.Lock()
        self.free: List[MmItemMemoryChunk] = [MmItemMemoryChunk((0, self.size), ShmSyncBuffer())]
        self.occupied: List[MmItemMemoryChunk] = []
        self._spare_flags: List[ShmSyncBuffer] = []
        self._stop = threading.Event()
        self._interval = recycle_interval_s
        self._thread: Optional[threading.Thread] = None
        if start_recycler:
            self._thread = threading.Thread(target=self._recycle_loop, name="mm-pool-recycler", daemon=True)
            self._thread.start()

    def _new_flag(self) -> ShmSyncBuffer:
        return self._spare_flags.pop() if self._spare_flags else ShmSyncBuffer()

    def get_slice_with_flag(self, src: torch.Tensor) -> Optional[Tuple[torch.Tensor, str]]:
        """Copy ``src`` into a free chunk; returns (view of the workspace, name of its sync flag) or None
        when no chunk is large enough (the caller then exports the tensor's own allocation)."""
        need = (src.numel() * src.element_size() + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        with self._lock:
            for i, ch in enumerate(self.free):
                if ch.mem_size >= need:
                    self.free.pop(i)
                    used = MmItemMemoryChunk((ch.start, ch.start + need), ch.sync_flag)
                    if ch.mem_size > need:
                        self.free.insert(i, MmItemMemoryChunk((ch.start + need, ch.end), self._new_flag()))
                    self.occupied.append(used)
                    break
            else:
                return None
        view = self.workspace[used.start: used.start + src.numel() * src.element_size()].view(src.dtype).view(src.shape)
        view.copy_(src, non_blocking=True)
        return view, used.sync_flag.name

    def recycle(self) -> int:
        """Return chunks whose consumers are done; merge adjacent free chunks.  Returns bytes freed."""
        freed = 0
        with self._lock:
            still = []
            for ch in self.occupied:
                if ch.try_to_recycle(self.num_consumers):
                    self.free.append(ch)
                    freed += ch.mem_size
                else:
                    still.append(ch)
            self.occupied = still
            self.free.sort(key=lambda c: c.start)
            merged: List[MmItemMemoryChunk] = []
            for ch in self.free:
                if merged and merged[-1].end == ch.start:
                    self._spare_flags.append(ch.sync_flag)
                    merged[-1] = MmItemMemoryChunk((merged[-1].start, ch.end), merged[-1].sync_flag)
                else:
                    merged.append(ch)
            self.free = merged
        return freed

    def free_bytes(self) -> int:
        with self._lock:
            return sum(c.mem_size for c in self.free)

    def _recycle_loop(self) -> None:
        while not self._stop.wait(self._interval):
            try:
                self.recycle()
            except Exception:  # pragma: no cover
                logger.exception("mm pool recycler failed")

    def shutdown(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        for ch in self.free + self.occupied:
            ch.sync_flag.close()
        for f in self._spare_flags:
            f.close()
        self.free, self.occupied, self._spare_flags = [], [], []


class CudaIpcTensorTransportProxy:
    """Pickle-friendly stand-in of a device tensor."""

    def __init__(self, tensor: torch.Tensor, sync_flag_name: Optional[str] = None) -> None:
        if not tensor.is_cuda:
            raise ValueError("CudaIpcTensorTransportProxy wraps CUDA tensors only")
        storage = tensor.untyped_storage()
        self.handle = storage._share_cuda_()
        self.shape, self.dtype, self.stride = tuple(tensor.shape), tensor.dtype, tuple(tensor.stride())
        self.storage_offset = tensor.storage_offset()
        self.sync_flag_name = sync_flag_name
        self._keepalive = tensor  # until pickled away / receiver done

    def __getstate__(self) -> Dict[str, Any]:
        d = dict(self.__dict__)
        d.pop("_keepalive", None)
        return d

    def __setstate__(self, state: Dict[str, Any]) -> None:
        self.__dict__.update(state)
        self._keepalive = None

    def reconstruct_on_device(self, device_index: Optional[int] = None) -> torch.Tensor:
        (dev, handle, size_bytes, offset_bytes, ref_handle, ref_offset, event_handle, event_sync) = self.handle
        target = dev if device_index is None else device_index
        with torch.cuda.device(target):
            storage = torch.UntypedStorage._new_shared_cuda(target, handle, size_bytes, offset_bytes, ref_handle,
                                                            ref_offset, event_handle, event_sync)
            mapped = torch.empty(0, dtype=self.dtype, device=f"cuda:{target}").set_(storage, self.storage_offset, self.shape,
                                                                                 self.stride)
            out = mapped.clone()  # receiver-owned copy: the sender's chunk can be recycled
            torch.cuda.current_stream().synchronize()
        if self.sync_flag_name:
            flag = ShmSyncBuffer.open(self.sync_flag_name)
            flag.signal()
            flag.close()
        return out


def wrap_mm_inputs(data: Any, pool: Optional[MmItemMemoryPool] = None) -> Any:
    """Replace every CUDA tensor in a nested dict / list / tuple by a transport proxy."""
    if isinstance(data, torch.Tensor):
        if not data.is_cuda:
            return data
        if pool is not None:
            got = pool.get_slice_with_flag(data)
            if got is not None:
                return CudaIpcTensorTransportProxy(got[0], got[1])
        return CudaIpcTensorTransportProxy(data.contiguous())
    if isinstance(data, dict):
        return {k: wrap_mm_inputs(v, pool) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(wrap_mm_inputs(v, pool) for v in data)
    return data


def unwrap_mm_inputs(data: Any, device_index: Optional[int] = None) -> Any:
    if isinstance(data, CudaIpcTensorTransportProxy):
        return data.reconstruct_on_device(device_index)
    if isinstance(data, dict):
        return {k: unwrap_mm_inputs(v, device_index) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return type(data)(unwrap_mm_inputs(v, device_index) for v in data)
    return data

"""``.mllm`` parameter files (V1 and V2) of the mllm C++ runtime: read through the memory-mapping C++
reader in ``csrc/host/mllm_file.cpp``, write V2 (mllm/core/schema/ModelFileV1.hpp:33-53,
ModelFileV2.hpp:11-59; Python writer of the reference: pymllm/mobile/convertor/model_file_v2.py).

Plain dtypes come back as tensors that view the mapping (copied on first device transfer); GGUF
block formats (Q4_0, Q8_0, Q4_K, Q6_K) are expanded to fp32 by the C++ thread pool and cast to
``gguf_dtype``.  V1 files carry no shapes: tensors come back flat and the model's loader reshapes
them to the parameter's shape."""

from __future__ import annotations

import warnings
from typing import Dict, Iterable, Iterator, Optional, Tuple

import numpy as np
import torch

from ..mem_cache.native import host_ext

# dtype ids of mllm/core/DataTypes.hpp
DTYPE_IDS: Dict[torch.dtype, int] = {
    torch.float32: 0, torch.float16: 1, torch.int8: 16, torch.int16: 17, torch.int32: 18,
    torch.bfloat16: 128, torch.uint8: 129, torch.int64: 132,
}
_ID_TO_DTYPE = {v: k for k, v in DTYPE_IDS.items()}
_ID_TO_DTYPE[134] = torch.uint8  # kByte
GGUF_IDS = {2: "Q4_0", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}


class MllmFileReader:
    def __init__(self, path: str) -> None:
        self._f = host_ext().MllmFile(str(path))

    @property
    def version(self) -> int:
        return int(self._f.version)

    @property
    def model_name(self) -> str:
        return self._f.model_name

    def names(self):
        return list(self._f.names())

    def info(self, name: str) -> Tuple[int, Tuple[int, ...], int, int]:
        dtype_id, shape, size, offset = self._f.info(name)
        return int(dtype_id), tuple(shape), int(size), int(offset)

    def tensor(self, name: str, gguf_dtype: torch.dtype = torch.bfloat16, threads: int = 0) -> torch.Tensor:
        dtype_id, shape, size, _ = self.info(name)
        if dtype_id in GGUF_IDS:
            t = torch.from_numpy(self._f.dequantize(name, threads)).to(gguf_dtype)
        elif dtype_id in _ID_TO_DTYPE:
            raw = self._f.raw(name)
            dt = _ID_TO_DTYPE[dtype_id]
            with warnings.catch_warnings():
                warnings.simplefilter("ignore", UserWarning)  # read-only mapping: callers copy on load
                t = torch.frombuffer(memoryview(raw), dtype=dt) if size else torch.empty(0, dtype=dt)
        else:
            raise ValueError(f"{name}: .mllm dtype id {dtype_id} is not supported "
                             f"(plain fp32/fp16/bf16/int8/int16/int32/int64/uint8 and GGUF {sorted(GGUF_IDS.values())} are)")
        return t.reshape(shape) if shape and int(np.prod(shape)) == t.numel() else t


def iter_mllm_tensors(path: str, gguf_dtype: torch.dtype = torch.bfloat16) -> Iterator[Tuple[str, torch.Tensor]]:
    r = MllmFileReader(path)
    for name in r.names():
        yield name, r.tensor(name, gguf_dtype)


def write_mllm(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], model_name: str = "") -> None:
    """Write a V2 file from ``(name, tensor)`` pairs (plain dtypes only)."""
    entries = []
    for name, t in tensors:
        t = t.detach().cpu().contiguous()
        if t.dtype not in DTYPE_IDS:
            raise ValueError(f"{name}: dtype {t.dtype} has no .mllm id")
        raw = t.view(torch.uint8).reshape(-1).numpy() if t.numel() else np.empty(0, dtype=np.uint8)
        entries.append((name, DTYPE_IDS[t.dtype], [int(s) for s in t.shape], raw))
    host_ext().write_mllm_v2(str(path), model_name, entries)


def write_mllm_v1(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Writer of the older layout (used by tests and for round trips with old runtimes)."""
    import struct

    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    table_len = sum(4 + len(n.encode()) + 8 + 8 + 4 for n, _ in items)
    off = 12 + table_len
    with open(path, "wb") as f:
        f.write(struct.pack("<iQ", 20012, table_len))
        blobs = []
        for n, t in items:
            raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
            nb = n.encode()
            f.write(struct.pack("<i", len(nb)) + nb + struct.pack("<QQi", len(raw), off, DTYPE_IDS[t.dtype]))
            blobs.append(raw)
            off += len(raw)
        for b in blobs:
            f.write(b)

"""A checkpoint tensor that is read only where it is used.

Under tensor / expert parallelism every rank keeps a slice of most matrices.  ``LazyTensor`` wraps a
safetensors slice handle: ``narrow`` and ``[...]`` read just the bytes of that slice from the file
(each rank reads 1/tp of a sharded matrix instead of all of it); anything else — ``copy_`` from it,
``reshape``, ``float`` ... — reads the whole tensor once and proceeds on the real tensor, so the weight
loaders do not need to know which kind they were given."""

from __future__ import annotations

from typing import Tuple

import torch

_ST_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
              "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
              "BOOL": torch.bool, "F8_E4M3": getattr(torch, "float8_e4m3fn", None), "F8_E5M2": getattr(torch, "float8_e5m2", None)}


class LazyTensor:
    bytes_read = 0  # process-wide tally of bytes fetched through lazy tensors (tests, load statistics)

    def __init__(self, st_slice, keepalive=None) -> None:
        self._slice = st_slice
        self._keepalive = keepalive     # the open file: handles must outlive buffered (name, tensor) pairs
        self._shape: Tuple[int, ...] = tuple(int(d) for d in st_slice.get_shape())
        self._dtype = _ST_DTYPES.get(str(st_slice.get_dtype()))
        self._full = None

    # ---- metadata: no read ----
    @property
    def shape(self) -> torch.Size:
        return torch.Size(self._shape)

    @property
    def dtype(self):
        return self._dtype if self._dtype is not None else self.materialize().dtype

    def dim(self) -> int:
        return len(self._shape)

    def size(self, d=None):
        return self.shape if d is None else self._shape[d]

    def numel(self) -> int:
        n = 1
        for d in self._shape:
            n *= d
        return n

    def is_floating_point(self) -> bool:
        return self.dtype.is_floating_point

    # ---- partial reads ----
    def _account(self, t: torch.Tensor) -> torch.Tensor:
        LazyTensor.bytes_read += t.numel() * t.element_size()
        return t

    def narrow(self, dim: int, start: int, length: int) -> torch.Tensor:
        if self._full is not None:
            return self._full.narrow(dim, start, length)
        dim = dim % len(self._shape)
        idx = tuple([slice(None)] * dim + [slice(int(start), int(start) + int(length))])
        return self._account(self._slice[idx])

    def __getitem__(self, idx) -> torch.Tensor:
        if self._full is not None:
            return self._full[idx]
        parts = idx if isinstance(idx, tuple) else (idx,)
        if all(isinstance(p, slice) and p.step in (None, 1) for p in parts):
            return self._account(self._slice[idx])
        return self.materialize()[idx]

    # ---- everything else: the whole tensor ----
    def materialize(self) -> torch.Tensor:
        if self._full is None:
            self._full = self._account(self._slice[:] if self._shape else self._slice[...])
        return self._full

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        return getattr(self.materialize(), name)

    def __len__(self) -> int:
        return self._shape[0]

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        def real(x):
            if isinstance(x, LazyTensor):
                return x.materialize()
            if isinstance(x, (list, tuple)):
                return type(x)(real(v) for v in x)
            return x

        return func(*real(args), **{k: real(v) for k, v in (kwargs or {}).items()})

    def __repr__(self) -> str:
        return f"LazyTensor(shape={self._shape}, dtype={self._dtype}, loaded={self._full is not None})"

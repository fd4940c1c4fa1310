"""Peer-mapped ("symmetric") buffers for the fused tensor-parallel kernels.

Each rank allocates the same buffers through ``torch.distributed._symmetric_memory`` (which
exchanges the handles and maps every peer's allocation into this process); the kernels then
read peers' partial sums and bump peers' flag counters with ordinary loads / stores /
reductions on those addresses.  ``TPComm`` owns, per process:

* two partial-sum buffers ``[max_rows, hidden]`` used alternately (the row-parallel GEMM writes
  straight into one of them, so there is no staging copy; the other may still be read by a
  slower rank);
* one flag block per partial buffer (``uint32 [max_rows][8]`` counters bumped by peers) and the
  local expected-count vector that goes with it.

When symmetric memory is not available (CPU / gloo ranks, a single GPU) ``TPComm.create``
returns ``None`` and callers use the collective of the process group instead.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist

from . import state as pstate

logger = logging.getLogger(__name__)
_FLAG_STRIDE = 8


@dataclass
class _Slot:
    data: torch.Tensor           # local [max_rows, hidden]
    flags: torch.Tensor          # local int32 [max_rows * 8]
    seq: torch.Tensor            # local int32 [max_rows] (not shared)
    data_ptrs: List[int] = field(default_factory=list)
    flag_ptrs: List[int] = field(default_factory=list)


class TPComm:
    def __init__(self, slots: List[_Slot], max_rows: int, hidden: int, dtype: torch.dtype, rank: int, world: int) -> None:
        self.slots = slots
        self.max_rows, self.hidden, self.dtype = max_rows, hidden, dtype
        self.rank, self.world = rank, world
        self._next = 0

    @classmethod
    def create(cls, hidden: int, dtype: torch.dtype, device: torch.device, max_rows: int = 256) -> Optional["TPComm"]:
        group = pstate.get_tp_group()
        if group.world_size == 1 or device.type != "cuda" or not dist.is_initialized():
            return None
        try:
            import torch.distributed._symmetric_memory as symm

            slots = []
            for _ in range(2):
                data = symm.empty((max_rows, hidden), dtype=dtype, device=device)
                flags = symm.empty((max_rows * _FLAG_STRIDE,), dtype=torch.int32, device=device)
                data.zero_()
                flags.zero_()
                hd = symm.rendezvous(data, group.group)
                hf = symm.rendezvous(flags, group.group)
                slots.append(_Slot(data=data, flags=flags, seq=torch.zeros(max_rows, dtype=torch.int32, device=device),
                                   data_ptrs=[int(p) for p in hd.buffer_ptrs], flag_ptrs=[int(p) for p in hf.buffer_ptrs]))
            torch.cuda.synchronize(device)
            group.barrier()
            return cls(slots, max_rows, hidden, dtype, group.rank_in_group, group.world_size)
        except Exception as exc:  # symmetric memory unsupported on this system
            logger.warning("symmetric memory unavailable (%s); tensor-parallel layers use NCCL collectives", exc)
            return None

    def partial_buffer(self, rows: int) -> Optional[torch.Tensor]:
        """The buffer the next row-parallel GEMM should write its partial sums into, or None when
        the batch is larger than the buffers (the caller then uses the group's all-reduce)."""
        if rows > self.max_rows:
            return None
        self._next ^= 1
        return self.slots[self._next].data[:rows]

    def slot_of(self, partial: torch.Tensor) -> Optional[_Slot]:
        for s in self.slots:
            if partial.data_ptr() == s.data.data_ptr():
                return s
        return None


_COMM: Optional[TPComm] = None


def get_tp_comm() -> Optional[TPComm]:
    return _COMM


def set_tp_comm(comm: Optional[TPComm]) -> None:
    global _COMM
    _COMM = comm

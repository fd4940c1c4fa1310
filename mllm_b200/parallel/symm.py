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

For prefill-sized batches (``create(..., prefill_rows=M)``) a second set of buffers carries the
sequence-sharded reduction: ``inbox [tp, M/tp, hidden]`` (every rank's GEMM epilogue stores the
partial-sum tiles of the rows this rank owns straight into it), ``hidden_full [M, hidden]`` (owners
store the normalised rows into every rank's copy) and two blocks of epoch flags.  All ranks issue
the same sequence of fused calls, so a per-process call counter (``epoch``) is the expected flag
value on every rank.

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


@dataclass
class PrefillBuffers:
    rows_cap: int                 # largest batch (token rows) the buffers hold; multiple of 128 * tp
    inbox: torch.Tensor           # local [tp, rows_cap / tp, hidden]
    tile_flags: torch.Tensor      # local int32 [(rows_cap / tp / 128) * 8]
    hidden_full: torch.Tensor     # local [rows_cap, hidden]
    gather_flags: torch.Tensor    # local int32 [rows_cap / 128]
    rs_count: torch.Tensor        # local int32 [rows_cap / 128]   (not shared)
    ag_count: torch.Tensor        # local int32 [rows_cap / tp / 128] (not shared)
    inbox_ptrs: List[int] = field(default_factory=list)
    tile_flag_ptrs: List[int] = field(default_factory=list)
    hidden_ptrs: List[int] = field(default_factory=list)
    gather_flag_ptrs: List[int] = field(default_factory=list)


class PrefillPartial:
    """Stands for the output of a row-parallel GEMM whose tiles went to the owners' inboxes; only
    the following norm (reduce-scatter + add + RMSNorm + all-gather) can consume it."""

    def __init__(self, rows: int, epoch: int, dtype: torch.dtype, device: torch.device) -> None:
        self.rows, self.epoch, self.dtype, self.device = rows, epoch, dtype, device


class TPComm:
    def __init__(self, slots: List[_Slot], max_rows: int, hidden: int, dtype: torch.dtype, rank: int, world: int,
                 prefill: Optional[PrefillBuffers] = None) -> None:
        self.slots = slots
        self.max_rows, self.hidden, self.dtype = max_rows, hidden, dtype
        self.rank, self.world = rank, world
        self._next = 0
        self.prefill = prefill
        self.epoch = 0                 # fused prefill calls issued so far (same on every rank)
        self.pending_gate: Optional[tuple] = None  # (epoch, rows) of a gather nobody has waited for yet
        self.prefill_fusion = True

    # ---- prefill ----
    def prefill_eligible(self, rows: int) -> bool:
        p = self.prefill
        return (p is not None and self.prefill_fusion and rows > self.max_rows and rows <= p.rows_cap
                and rows % (128 * self.world) == 0)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    @classmethod
    def create(cls, hidden: int, dtype: torch.dtype, device: torch.device, max_rows: int = 256,
               prefill_rows: int = 0) -> Optional["TPComm"]:
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
            prefill = None
            tp = group.world_size
            if prefill_rows > 0:
                cap = (prefill_rows + 128 * tp - 1) // (128 * tp) * (128 * tp)
                own = cap // tp
                inbox = symm.empty((tp, own, hidden), dtype=dtype, device=device)
                tile_flags = symm.empty((own // 128 * _FLAG_STRIDE,), dtype=torch.int32, device=device)
                hidden_full = symm.empty((cap, hidden), dtype=dtype, device=device)
                gather_flags = symm.empty((cap // 128,), dtype=torch.int32, device=device)
                for t in (inbox, tile_flags, hidden_full, gather_flags):
                    t.zero_()
                handles = [symm.rendezvous(t, group.group) for t in (inbox, tile_flags, hidden_full, gather_flags)]
                prefill = PrefillBuffers(
                    rows_cap=cap, inbox=inbox, tile_flags=tile_flags, hidden_full=hidden_full, gather_flags=gather_flags,
                    rs_count=torch.zeros(cap // 128, dtype=torch.int32, device=device),
                    ag_count=torch.zeros(own // 128, dtype=torch.int32, device=device),
                    inbox_ptrs=[int(p) for p in handles[0].buffer_ptrs],
                    tile_flag_ptrs=[int(p) for p in handles[1].buffer_ptrs],
                    hidden_ptrs=[int(p) for p in handles[2].buffer_ptrs],
                    gather_flag_ptrs=[int(p) for p in handles[3].buffer_ptrs])
            torch.cuda.synchronize(device)
            group.barrier()
            return cls(slots, max_rows, hidden, dtype, group.rank_in_group, group.world_size, prefill)
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

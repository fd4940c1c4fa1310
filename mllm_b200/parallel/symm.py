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

All of these live in one :class:`SymmetricHeap`: a single peer-mapped allocation per rank (one
rendezvous), carved up by a deterministic host-side offset allocator (C++), so a buffer's address on
rank ``r`` is that rank's heap base plus the same offset.

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
_HEAP_ALIGN = 256
_GUARD = 256          # canary bytes in front of and behind every heap block
_GUARD_BYTE = 0xA5


class SymmetricHeap:
    """One byte buffer per rank, mapped into every peer, plus the offset allocator that carves it.

    Every rank must make the same ``tensor`` / ``free`` calls in the same order (the allocator is
    deterministic), which gives every buffer the same offset on every rank.  Each block sits between two
    runs of canary bytes; :meth:`check_guards` tells whether a kernel (local or a peer's) wrote outside a
    buffer — the multi-rank tests call it after their collectives."""

    def __init__(self, buf: torch.Tensor, base_ptrs: List[int]) -> None:
        from ..mem_cache.native import host_ext

        assert buf.dtype == torch.uint8 and buf.dim() == 1
        self.buf = buf
        self.base_ptrs = [int(p) for p in base_ptrs]
        self.alloc = host_ext().SymmHeapAllocator(int(buf.numel()), _HEAP_ALIGN)
        self._offsets = {}

    @classmethod
    def create(cls, nbytes: int, device: torch.device, group) -> "SymmetricHeap":
        """Collective over ``group``: allocates, zeroes and exchanges the mappings once."""
        import os

        # The kernels of this build reach peers with plain loads / stores / reductions only.  Ask the
        # symmetric-memory layer not to bind the heap to an NVLink multicast object as well: nothing here
        # would use it, it is one more collective set-up step per rank, and memory bound to such an
        # object makes a rank's abnormal exit visible as NVLink faults on its peers.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        buf = symm.empty((int(nbytes),), dtype=torch.uint8, device=device)
        buf.zero_()
        handle = symm.rendezvous(buf, group)
        return cls(buf, [int(p) for p in handle.buffer_ptrs])

    @classmethod
    def local(cls, nbytes: int, world: int = 1, device="cpu") -> "SymmetricHeap":
        """A heap without peers (tests, single rank): every "peer" base is the local buffer."""
        buf = torch.zeros(int(nbytes), dtype=torch.uint8, device=device)
        return cls(buf, [buf.data_ptr()] * world)

    @staticmethod
    def bytes_for(shapes_dtypes) -> int:
        """Capacity that fits the given ``(shape, dtype)`` buffers, each rounded to the heap alignment."""
        total = 0
        for shape, dtype in shapes_dtypes:
            n = torch.empty((), dtype=dtype).element_size()
            for d in shape:
                n *= int(d)
            total += (n + 2 * _GUARD + _HEAP_ALIGN - 1) // _HEAP_ALIGN * _HEAP_ALIGN
        return total

    def tensor(self, shape, dtype: torch.dtype):
        """A zero-copy view of a fresh block, and its address on every rank."""
        n = torch.empty((), dtype=dtype).element_size()
        for d in shape:
            n *= int(d)
        blk = int(self.alloc.alloc(n + 2 * _GUARD))
        if blk < 0:
            raise MemoryError(f"symmetric heap: no room for {n} bytes ({self.alloc.used} of {self.alloc.capacity} used)")
        off = blk + _GUARD
        self.buf[blk:off] = _GUARD_BYTE
        self.buf[off + n:off + n + _GUARD] = _GUARD_BYTE
        t = self.buf[off:off + n].view(dtype).view(*shape)
        self._offsets[t.data_ptr()] = (blk, n)
        return t, [b + off for b in self.base_ptrs]

    def check_guards(self) -> List[int]:
        """Offsets of the live buffers whose canary bytes were overwritten (empty: all intact)."""
        bad = []
        for blk, n in self._offsets.values():
            front = self.buf[blk:blk + _GUARD]
            back = self.buf[blk + _GUARD + n:blk + 2 * _GUARD + n]
            if bool((front != _GUARD_BYTE).any()) or bool((back != _GUARD_BYTE).any()):
                bad.append(blk + _GUARD)
        return bad

    def free(self, t: torch.Tensor) -> None:
        entry = self._offsets.pop(t.data_ptr(), None)
        if entry is None or not self.alloc.free(entry[0]):
            raise ValueError("tensor does not start a block of this heap")


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


class PrefillShard:
    """The rows this rank owns of a block's output, already complete (no partial sums left to add): what the
    expert-parallel exchange returns.  Only the following norm (add + RMSNorm + all-gather) can consume it."""

    def __init__(self, rows: int, epoch: int, shard: torch.Tensor) -> None:
        self.rows, self.epoch, self.shard = rows, epoch, shard
        self.dtype, self.device = shard.dtype, shard.device


class EPComm:
    """Peer-mapped buffers of the expert-parallel token exchange (``csrc/ep_a2a.cu``): every rank's per-expert
    pair counts, the receive slab for routed token rows (grouped by local expert, then by source rank), the
    (source rank, pair) note beside each row, the return buffer for the experts' output rows, and three flag
    blocks (counts, dispatch, return) holding the epoch of the last completed exchange per source rank."""

    def __init__(self, heap: "SymmetricHeap", rank: int, world: int, hidden: int, dtype: torch.dtype, experts: int,
                 top_k: int, tokens_cap: int, slab_factor: float = 2.0) -> None:
        i32 = torch.int32
        self.rank, self.world, self.hidden, self.dtype = rank, world, hidden, dtype
        self.experts, self.top_k = experts, top_k
        self.tokens_cap = int(tokens_cap)                 # tokens of ONE rank per call
        self.pairs_cap = self.tokens_cap * top_k
        # rows a rank receives: pairs of all ranks / ranks on average; the factor is head-room for skewed routing
        self.cap_rows = int(min(self.pairs_cap * world, max(256, slab_factor * self.pairs_cap)))
        self.cap_rows = (self.cap_rows + 127) // 128 * 128
        dev = heap.buf.device
        cut = {}
        for name, shape, dt in (("cnt_all", (world * experts,), i32), ("cnt_flags", (8,), i32),
                                ("recv_x", (self.cap_rows, hidden), dtype), ("recv_meta", (self.cap_rows, 2), i32),
                                ("disp_flags", (8,), i32), ("ret_y", (self.pairs_cap, hidden), dtype),
                                ("ret_flags", (8,), i32)):
            cut[name] = heap.tensor(shape, dt)
        self.recv_x, self.ret_y = cut["recv_x"][0], cut["ret_y"][0]
        self.disp_flags, self.ret_flags = cut["disp_flags"][0], cut["ret_flags"][0]
        self.ptrs = [cut[n][1] for n in ("cnt_all", "cnt_flags", "recv_x", "recv_meta", "disp_flags", "ret_y", "ret_flags")]
        self.heap = heap
        self.epoch = 0
        # local scratch of the plan
        el = experts // world
        self.pair_dst_rank = torch.empty(self.pairs_cap, dtype=i32, device=dev)
        self.pair_dst_row = torch.empty(self.pairs_cap, dtype=i32, device=dev)
        self.expert_offsets = torch.zeros(el + 1, dtype=i32, device=dev)
        self.work = torch.zeros((el + self.cap_rows // 16 + 1, 2), dtype=i32, device=dev)
        self.n_work = torch.zeros(1, dtype=i32, device=dev)
        self.recv_rows = torch.zeros(1, dtype=i32, device=dev)
        self.done = torch.zeros(2, dtype=i32, device=dev)
        self.pair_index = torch.arange(self.pairs_cap, dtype=i32, device=dev)

    @staticmethod
    def heap_bytes(hidden: int, dtype: torch.dtype, world: int, experts: int, top_k: int, tokens_cap: int,
                   slab_factor: float = 2.0) -> int:
        pairs = tokens_cap * top_k
        cap = int(min(pairs * world, max(256, slab_factor * pairs)))
        cap = (cap + 127) // 128 * 128
        i32 = torch.int32
        return SymmetricHeap.bytes_for([((world * experts,), i32), ((8,), i32), ((cap, hidden), dtype), ((cap, 2), i32),
                                        ((8,), i32), ((pairs, hidden), dtype), ((8,), i32)])

    def eligible(self, tokens_total: int) -> bool:
        """Prefill-sized batches whose rows split evenly into whole 128-row tiles per rank."""
        return (tokens_total % (128 * self.world) == 0 and 0 < tokens_total // self.world <= self.tokens_cap)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


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

    @staticmethod
    def _plan(hidden: int, dtype: torch.dtype, tp: int, max_rows: int, prefill_rows: int):
        """Shapes of the shared buffers in allocation order, plus (rows_cap, rows per owner)."""
        i32 = torch.int32
        plan = [((max_rows, hidden), dtype), ((max_rows * _FLAG_STRIDE,), i32)] * 2
        cap = own = 0
        if prefill_rows > 0:
            cap = (prefill_rows + 128 * tp - 1) // (128 * tp) * (128 * tp)
            own = cap // tp
            plan += [((tp, own, hidden), dtype), ((own // 128 * _FLAG_STRIDE,), i32), ((cap, hidden), dtype),
                     ((cap // 128,), i32)]
        return plan, cap, own

    @classmethod
    def heap_bytes(cls, hidden: int, dtype: torch.dtype, tp: int, max_rows: int = 256, prefill_rows: int = 0) -> int:
        return SymmetricHeap.bytes_for(cls._plan(hidden, dtype, tp, max_rows, prefill_rows)[0])

    @classmethod
    def from_heap(cls, heap: SymmetricHeap, hidden: int, dtype: torch.dtype, device, rank: int, tp: int,
                  max_rows: int = 256, prefill_rows: int = 0) -> "TPComm":
        """Carves the buffers out of a (zeroed) heap; every rank calls this with the same arguments."""
        i32 = torch.int32
        plan, cap, own = cls._plan(hidden, dtype, tp, max_rows, prefill_rows)
        cut = [heap.tensor(shape, dt) for shape, dt in plan]
        slots = [_Slot(data=cut[2 * i][0], flags=cut[2 * i + 1][0], seq=torch.zeros(max_rows, dtype=i32, device=device),
                       data_ptrs=cut[2 * i][1], flag_ptrs=cut[2 * i + 1][1]) for i in range(2)]
        prefill = None
        if prefill_rows > 0:
            (inbox, inbox_ptrs), (tile_flags, tile_flag_ptrs), (hidden_full, hidden_ptrs), (gather_flags, gather_flag_ptrs) = cut[4:8]
            prefill = PrefillBuffers(
                rows_cap=cap, inbox=inbox, tile_flags=tile_flags, hidden_full=hidden_full, gather_flags=gather_flags,
                rs_count=torch.zeros(cap // 128, dtype=i32, device=device),
                ag_count=torch.zeros(own // 128, dtype=i32, device=device),
                inbox_ptrs=inbox_ptrs, tile_flag_ptrs=tile_flag_ptrs, hidden_ptrs=hidden_ptrs,
                gather_flag_ptrs=gather_flag_ptrs)
        comm = cls(slots, max_rows, hidden, dtype, rank, tp, prefill)
        comm.heap = heap
        return comm

    @classmethod
    def create(cls, hidden: int, dtype: torch.dtype, device: torch.device, max_rows: int = 256,
               prefill_rows: int = 0) -> Optional["TPComm"]:
        group = pstate.get_tp_group()
        if group.world_size == 1 or device.type != "cuda" or not dist.is_initialized():
            return None
        try:
            tp = group.world_size
            heap = SymmetricHeap.create(cls.heap_bytes(hidden, dtype, tp, max_rows, prefill_rows), device, group.group)
            comm = cls.from_heap(heap, hidden, dtype, device, group.rank_in_group, tp, max_rows, prefill_rows)
            torch.cuda.synchronize(device)
            group.barrier()
            return comm
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
_EP_COMM: Optional[EPComm] = None


def get_ep_comm() -> Optional[EPComm]:
    return _EP_COMM


def set_ep_comm(comm: Optional[EPComm]) -> None:
    global _EP_COMM
    _EP_COMM = comm


def get_tp_comm() -> Optional[TPComm]:
    return _COMM


def set_tp_comm(comm: Optional[TPComm]) -> None:
    global _COMM
    _COMM = comm

"""KV-cache storage and the two index pools that map requests to it.

Three objects, with the roles of pymllm/mem_cache/memory_pool.py:23-415:

* :class:`KVPool` — the K and V rows of every layer, addressed by *slot*
  (one slot = one token position of one request).  Slots are grouped into
  pages of ``page_size`` consecutive slots; page 0 is never handed out, so
  slot 0 is a safe sink for padded batch entries under CUDA graphs.
* :class:`TokenToKVPoolAllocator` — hands out and takes back slots (whole
  pages when ``page_size > 1``).  The free list lives on the host: the
  scheduler that calls it is host code, and a step only needs one small
  host-to-device copy of the slots it was given.
* :class:`ReqToTokenPool` — a ``[max_reqs, max_context]`` int32 table on the
  device; row ``r`` lists the slots of request ``r`` in position order.  The
  attention kernels read this table directly, so no flat index list is built
  per step.

All K/V rows of all layers sit in ONE allocation laid out
``[layer, k|v, kv_head, slot, head_dim]`` (head-major), so that a kernel gets a layer's
buffers as base pointer + strides and 180 GB of HBM is carved exactly once.  Head-major
means that consecutive slots of one KV head are consecutive 256-byte rows: a page, or any
run of slots a request was given in one piece, is one contiguous block per head, which the
attention kernels fetch as whole TMA boxes instead of row by row.  ``get_kv_buffer``
hands out ``[slot, kv_head, head_dim]`` *views* of that storage, so code that indexes the
cache by slot does not see the difference.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch


class KVPool:
    def __init__(
        self,
        size: int,
        layer_num: int,
        kv_heads: int,
        head_dim: int,
        dtype: torch.dtype,
        device: torch.device | str,
        page_size: int = 1,
        v_head_dim: Optional[int] = None,
        layer_offset: int = 0,
    ) -> None:
        # ``layer_offset``: global index of the first layer held here (a pipeline stage keeps K/V only for its
        # own layers, which address the pool by their global index)
        self.layer_offset = int(layer_offset)
        if v_head_dim is not None and v_head_dim != head_dim:
            raise ValueError("K and V head widths must match in this pool")
        self.page_size = int(page_size)
        # usable slots rounded down to whole pages, plus the reserved page 0
        self.size = (int(size) // self.page_size) * self.page_size
        self.num_slots = self.size + self.page_size
        self.layer_num = layer_num
        self.kv_heads = kv_heads
        self.head_dim = head_dim
        self.dtype = dtype
        self.device = torch.device(device)
        self.store = torch.zeros(
            (layer_num, 2, kv_heads, self.num_slots, head_dim), dtype=dtype, device=self.device
        )
        self.k_buffer: List[torch.Tensor] = [self.store[l, 0].transpose(0, 1) for l in range(layer_num)]
        self.v_buffer: List[torch.Tensor] = [self.store[l, 1].transpose(0, 1) for l in range(layer_num)]

    @staticmethod
    def cell_bytes(layer_num: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> int:
        """Bytes one token occupies over all layers (K and V)."""
        return 2 * layer_num * kv_heads * head_dim * torch.empty((), dtype=dtype).element_size()

    def get_key_buffer(self, layer_id: int) -> torch.Tensor:
        return self.k_buffer[layer_id - self.layer_offset]

    def get_value_buffer(self, layer_id: int) -> torch.Tensor:
        return self.v_buffer[layer_id - self.layer_offset]

    def get_kv_buffer(self, layer_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.k_buffer[layer_id - self.layer_offset], self.v_buffer[layer_id - self.layer_offset]

    def set_kv_buffer(self, layer_id: int, loc: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        """Scatter rows ``k[i]``/``v[i]`` to slot ``loc[i]``.

        The model's fused QK-norm + RoPE kernel normally writes the cache itself;
        this entry is the stand-alone form (same contract as the reference's
        ``store_cache``: exact copy, later rows win on duplicate slots).
        """
        from ..ops import kv_write

        kv_write(
            k.view(-1, self.kv_heads, self.head_dim),
            v.view(-1, self.kv_heads, self.head_dim),
            loc,
            self.k_buffer[layer_id - self.layer_offset],
            self.v_buffer[layer_id - self.layer_offset],
        )

    def clear(self) -> None:
        self.store.zero_()


class TokenToKVPoolAllocator:
    """Host-side free list of KV slots / pages.

    ``alloc(n)`` returns ``n`` slot ids as an int64 tensor on ``device`` (or
    ``None`` when there is not enough room — the caller then evicts from the
    prefix cache and retries).  With ``page_size > 1`` slots are granted in
    whole pages: ``alloc`` rounds up to pages, and ``free`` returns a page once
    any of its slots is freed — callers free page-aligned runs.
    """

    def __init__(self, size: int, page_size: int = 1, device: torch.device | str = "cpu") -> None:
        self.page_size = int(page_size)
        self.num_pages = int(size) // self.page_size
        self.size = self.num_pages * self.page_size
        self.device = torch.device(device)
        self._groups: Optional[List[np.ndarray]] = None
        self.clear()

    def clear(self) -> None:
        # page ids 1..num_pages (page 0 is the padding sink)
        self._free = np.arange(1, self.num_pages + 1, dtype=np.int64)
        self._released: List[np.ndarray] = []
        self._groups = None

    def available_size(self) -> int:
        return (len(self._free) + sum(len(r) for r in self._released)) * self.page_size

    def _merge_released(self) -> None:
        if self._released:
            merged = np.concatenate([self._free] + self._released)
            self._free = np.unique(merged)  # sorted: keeps grants contiguous over time
            self._released = []

    def alloc_host(self, need_size: int) -> Optional[np.ndarray]:
        """Slot ids as a numpy int64 array, or None if the pool is short."""
        if need_size <= 0:
            return np.empty((0,), dtype=np.int64)
        pages = -(-need_size // self.page_size)
        if pages > len(self._free):
            self._merge_released()
            if pages > len(self._free):
                return None
        got, self._free = self._free[:pages], self._free[pages:]
        if self.page_size == 1:
            return got.copy()
        slots = (got[:, None] * self.page_size + np.arange(self.page_size, dtype=np.int64)[None, :]).reshape(-1)
        return slots[:need_size] if need_size % self.page_size == 0 else slots[:need_size].copy()

    def alloc(self, need_size: int) -> Optional[torch.Tensor]:
        host = self.alloc_host(need_size)
        if host is None:
            return None
        t = torch.from_numpy(host)
        return t.to(self.device, non_blocking=True) if self.device.type != "cpu" else t

    def free(self, indices) -> None:
        if indices is None:
            return
        if isinstance(indices, torch.Tensor):
            if indices.numel() == 0:
                return
            indices = indices.detach().to("cpu", torch.int64).numpy()
        arr = np.asarray(indices, dtype=np.int64).reshape(-1)
        if arr.size == 0:
            return
        pages = arr if self.page_size == 1 else np.unique(arr // self.page_size)
        pages = pages[pages > 0]
        if self._groups is not None:
            self._groups.append(pages)
        else:
            self._released.append(pages)

    # batched frees: collect, then release once
    def free_group_begin(self) -> None:
        self._groups = []

    def free_group_end(self) -> None:
        groups, self._groups = self._groups, None
        if groups:
            self._released.append(np.concatenate(groups))


class GDNPool:
    """Per-request state of the gated-delta-net layers of a hybrid model: the fp32 recurrent matrix
    ``[layers, rows, Hv, Dk, Dv]`` and the last ``K-1`` convolution inputs ``[layers, rows, C, K-1]``.
    A request uses the row of its ``req_to_token`` slot, so no separate allocator is needed for the
    first ``slots`` rows; ``track_slots`` further rows hold snapshots that the hybrid prefix cache
    keeps at the ends of cached prefixes (role of pymllm/mem_cache/memory_pool.py:479-631)."""

    def __init__(self, num_layers: int, slots: int, num_v_heads: int, head_k_dim: int, head_v_dim: int, conv_dim: int,
                 conv_kernel: int, device, conv_dtype: torch.dtype = torch.bfloat16, track_slots: int = 0) -> None:
        self.num_layers, self.slots, self.track_slots = num_layers, slots, int(track_slots)
        rows = slots + self.track_slots
        self.recurrent = torch.zeros((num_layers, rows, num_v_heads, head_k_dim, head_v_dim), dtype=torch.float32, device=device)
        self.conv = torch.zeros((num_layers, rows, conv_dim, conv_kernel - 1), dtype=conv_dtype, device=device)
        self._free_track: List[int] = list(range(slots, rows))

    def layer(self, idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.recurrent[idx], self.conv[idx]

    def reset(self, slot) -> None:
        self.recurrent[:, slot] = 0
        self.conv[:, slot] = 0

    def copy(self, src: int, dst: int) -> None:
        self.recurrent[:, dst] = self.recurrent[:, src]
        self.conv[:, dst] = self.conv[:, src]

    copy_states = copy

    # ---- snapshot rows ----
    def track_available(self) -> int:
        return len(self._free_track)

    def alloc_track_slot(self) -> Optional[int]:
        return self._free_track.pop() if self._free_track else None

    def free_track_slot(self, slot: int) -> None:
        slot = int(slot)
        if not (self.slots <= slot < self.slots + self.track_slots) or slot in self._free_track:
            raise ValueError(f"row {slot} is not an allocated snapshot row")
        self._free_track.append(slot)

    def bytes(self) -> int:
        return self.recurrent.numel() * 4 + self.conv.numel() * self.conv.element_size()


class ReqToTokenPool:
    """Request slot -> KV slot table (device) plus a host free list of request slots.

    The table has one row more than ``max_reqs``: row ``pad_row`` is never handed out.  Batches padded
    up to a captured CUDA-graph size point their extra rows at it, so kernels that keep per-request
    state by request row (recurrent / convolution state of hybrid models) read and write a row no
    request owns; its KV entries stay 0, the reserved sink slot of the KV pool."""

    def __init__(self, max_reqs: int, max_context_len: int, device: torch.device | str) -> None:
        self.size = int(max_reqs)
        self.max_context_len = int(max_context_len)
        self.device = torch.device(device)
        self.pad_row = self.size
        self.req_to_token = torch.zeros(
            (self.size + 1, self.max_context_len), dtype=torch.int32, device=self.device
        )
        self.free_slots: List[int] = list(range(self.size))

    def available_size(self) -> int:
        return len(self.free_slots)

    def alloc(self, need_size: int) -> Optional[List[int]]:
        if need_size > len(self.free_slots):
            return None
        out, self.free_slots = self.free_slots[:need_size], self.free_slots[need_size:]
        return out

    def free(self, slot) -> None:
        if isinstance(slot, int):
            self.free_slots.append(slot)
        else:
            self.free_slots.extend(int(s) for s in slot)

    def write(self, index, values: torch.Tensor) -> None:
        self.req_to_token[index] = values.to(self.req_to_token.dtype)

    def clear(self) -> None:
        self.free_slots = list(range(self.size))

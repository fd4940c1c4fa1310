"""C++ twins of the host-side cache structures (``mllm_b200/csrc/host``): the slot allocator of the
paged KV pool and the page-aligned radix prefix tree, behind the same interfaces as the Python
versions in ``memory_pool.py`` / ``radix_cache.py`` (roles of pymllm/mem_cache/memory_pool.py:165-317
and radix_cache.py:223-460).  The scheduler loop touches these structures for every request of every
step, so they are the part of the host path worth keeping out of the interpreter."""

from __future__ import annotations

from typing import Any, Callable, Optional

import numpy as np
import torch

from .._build import load_extension
from .base_prefix_cache import BasePrefixCache, EvictResult, InsertResult, MatchResult, RadixKey, hash_bytes

_EMPTY = np.empty(0, dtype=np.int64)


def host_ext():
    mod = load_extension("mllm_b200_host")
    if mod is None:
        raise RuntimeError("the mllm_b200_host extension is not built")
    return mod


def _extra(extra_key: Optional[str]) -> int:
    if extra_key is None:
        return 0
    h = hash_bytes(str(extra_key).encode()) & 0xFFFFFFFFFFFFFFFF
    return h - (1 << 64) if h >= (1 << 63) else h      # the tree takes a signed 64-bit key


class NativeTokenToKVPoolAllocator:
    """Drop-in replacement of ``TokenToKVPoolAllocator`` backed by ``PageAllocator`` (C++)."""

    def __init__(self, size: int, page_size: int = 1, device: torch.device | str = "cpu") -> None:
        self.size, self.page_size, self.device = int(size), int(page_size), torch.device(device)
        # the Python allocator owns slots 1..size (slot 0 is padding): same here, in pages
        self._impl = host_ext().PageAllocator(self.size + self.page_size, self.page_size)

    def clear(self) -> None:
        self._impl.clear()

    def available_size(self) -> int:
        return int(self._impl.available())

    def alloc_host(self, need_size: int) -> Optional[np.ndarray]:
        return self._impl.alloc(int(need_size))

    def alloc(self, need_size: int) -> Optional[torch.Tensor]:
        out = self.alloc_host(need_size)
        if out is None:
            return None
        t = torch.from_numpy(out)
        return t if self.device.type == "cpu" else t.pin_memory().to(self.device, non_blocking=True)

    def free(self, indices) -> None:
        if isinstance(indices, torch.Tensor):
            indices = indices.detach().to("cpu", torch.int64).numpy()
        self._impl.free(np.ascontiguousarray(indices, dtype=np.int64))

    def free_group_begin(self) -> None:
        self._impl.group_begin()

    def free_group_end(self) -> None:
        self._impl.group_end()


class NativeRadixCache(BasePrefixCache):
    """``RadixCache`` interface over the C++ ``RadixTree``; node handles are integer ids."""

    def __init__(self, token_to_kv_pool_allocator=None, page_size: int = 1,
                 on_evict: Optional[Callable[[np.ndarray], None]] = None, disable: bool = False) -> None:
        self.allocator = token_to_kv_pool_allocator
        self.page_size = int(page_size)
        self.on_evict = on_evict
        self.disable = disable
        self._tree = host_ext().RadixTree(self.page_size)
        self.root = 0

    def reset(self) -> None:
        self._tree.reset()

    def evictable_size(self) -> int:
        return int(self._tree.evictable_size())

    def protected_size(self) -> int:
        return int(self._tree.protected_size())

    def total_size(self) -> int:
        return int(self._tree.total_size())

    def match_prefix(self, key: RadixKey) -> MatchResult:
        if self.disable or len(key) < self.page_size:
            return MatchResult(indices=_EMPTY, last_node=self.root, prefix_len=0)
        slots, node = self._tree.match_prefix(np.asarray(key.token_ids, dtype=np.int64), _extra(key.extra_key))
        return MatchResult(indices=slots, last_node=int(node), prefix_len=len(slots))

    def insert(self, key: RadixKey, value=None, **kw) -> InsertResult:
        if self.disable:
            return InsertResult(prefix_len=0, last_node=self.root)
        tokens = np.asarray(key.token_ids, dtype=np.int64)
        if value is None:
            value = tokens
        elif isinstance(value, torch.Tensor):
            value = value.detach().to("cpu", torch.int64).numpy()
        value = np.ascontiguousarray(value, dtype=np.int64)
        n = len(tokens) - len(tokens) % self.page_size
        prefix, last = self._tree.insert(tokens[:n], value[:n], _extra(key.extra_key))
        return InsertResult(prefix_len=int(prefix), last_node=int(last))

    def inc_lock_ref(self, node: Any):
        if self.disable or node is None:
            return 0
        before = self._tree.evictable_size()
        self._tree.inc_lock_ref(int(node))
        return int(self._tree.evictable_size() - before)

    def dec_lock_ref(self, node: Any, **kw):
        if self.disable or node is None:
            return 0
        before = self._tree.evictable_size()
        self._tree.dec_lock_ref(int(node))
        return int(self._tree.evictable_size() - before)

    def evict(self, num_tokens: int, swa_num_tokens: int = 0) -> EvictResult:
        if self.disable or num_tokens <= 0:
            return EvictResult()
        freed = self._tree.evict(int(num_tokens))
        if len(freed):
            if self.on_evict is not None:
                self.on_evict(freed)
            if self.allocator is not None:
                self.allocator.free(freed)
        return EvictResult(full_evicted=int(len(freed)))

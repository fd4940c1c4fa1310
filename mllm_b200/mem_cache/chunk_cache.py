"""Prefix cache that never matches: used when radix reuse is switched off
(role of pymllm/mem_cache/chunk_cache.py:23-74)."""

from __future__ import annotations

import numpy as np

from .base_prefix_cache import BasePrefixCache, EvictResult, InsertResult, MatchResult, RadixKey


class ChunkCache(BasePrefixCache):
    def __init__(self, token_to_kv_pool_allocator=None, page_size: int = 1) -> None:
        self.allocator = token_to_kv_pool_allocator
        self.page_size = page_size

    def reset(self) -> None:
        pass

    def match_prefix(self, key: RadixKey) -> MatchResult:
        return MatchResult(indices=np.empty((0,), dtype=np.int64), last_node=None, prefix_len=0)

    def insert(self, key: RadixKey, value=None, **kw) -> InsertResult:
        return InsertResult(prefix_len=0, last_node=None)

    def evict(self, num_tokens: int, swa_num_tokens: int = 0) -> EvictResult:
        return EvictResult()

    def inc_lock_ref(self, node):
        return None

    def dec_lock_ref(self, node, **kw):
        return None

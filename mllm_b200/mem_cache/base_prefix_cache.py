"""Types shared by the prefix caches (roles of pymllm/mem_cache/base_prefix_cache.py:23-206)."""

from __future__ import annotations

import hashlib
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np


def hash_token_ids(token_ids: Sequence[Union[int, Tuple[int, ...]]], prior_hash: Optional[str] = None) -> str:
    """SHA-256 over one page of token ids, chained on the previous page's digest."""
    h = hashlib.sha256()
    if prior_hash:
        h.update(bytes.fromhex(prior_hash))
    for t in token_ids:
        if isinstance(t, tuple):
            for x in t:
                h.update(int(x).to_bytes(4, "little", signed=False))
        else:
            h.update(int(t).to_bytes(4, "little", signed=False))
    return h.hexdigest()


def hash_to_int64(hex_str: str) -> int:
    v = int(hex_str[:16], 16)
    return v - (1 << 64) if v >= (1 << 63) else v


def hash_bytes(data: bytes) -> int:
    return int.from_bytes(hashlib.sha256(data).digest()[:8], "little", signed=False)


class RadixKey:
    """Token ids plus an optional namespace (``extra_key``: LoRA id, image hash, ...)."""

    __slots__ = ("token_ids", "extra_key")

    def __init__(self, token_ids: Sequence[int], extra_key: Optional[str] = None) -> None:
        self.token_ids = token_ids if isinstance(token_ids, list) else list(token_ids)
        self.extra_key = extra_key

    def __len__(self) -> int:
        return len(self.token_ids)

    def __iter__(self) -> Iterator[int]:
        return iter(self.token_ids)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return RadixKey(self.token_ids[idx], self.extra_key)
        return RadixKey([self.token_ids[idx]], self.extra_key)

    def __repr__(self) -> str:
        head = self.token_ids[:8]
        return f"RadixKey(extra_key={self.extra_key!r}, n={len(self.token_ids)}, head={head})"


@dataclass
class MatchResult:
    indices: np.ndarray  # int64 KV slots of the matched prefix
    last_node: Any = None
    prefix_len: int = 0
    mamba_branching_seqlen: Optional[int] = None
    state_slot: Optional[int] = None  # hybrid models: snapshot row holding the state at the end of the prefix


@dataclass
class InsertResult:
    prefix_len: int = 0  # tokens that were already in the tree
    last_node: Any = None
    mamba_exist: bool = False
    adopted: int = 0  # tokens whose slots the tree took over in place of older ones (revived tombstones)


@dataclass
class EvictResult:
    full_evicted: int = 0
    swa_evicted: int = 0
    mamba_evicted: int = 0


class BasePrefixCache(ABC):
    @abstractmethod
    def reset(self) -> None: ...

    @abstractmethod
    def match_prefix(self, key: RadixKey) -> MatchResult: ...

    @abstractmethod
    def insert(self, key: RadixKey, value=None, **kw) -> InsertResult: ...

    @abstractmethod
    def evict(self, num_tokens: int, swa_num_tokens: int = 0) -> EvictResult: ...

    @abstractmethod
    def inc_lock_ref(self, node: Any): ...

    @abstractmethod
    def dec_lock_ref(self, node: Any, **kw): ...

    def evictable_size(self) -> int:
        return 0

    def protected_size(self) -> int:
        return 0

    def total_size(self) -> int:
        return 0

    def pretty_print(self) -> None:
        pass

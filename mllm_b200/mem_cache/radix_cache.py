"""Radix-tree prefix cache over KV slots (host side).

Behavioural contract of pymllm/mem_cache/radix_cache.py:129-530:

* keys are token-id sequences (namespaced by ``extra_key``); a node stores the
  KV slots of its edge label;
* matching and insertion work on whole pages: lengths are rounded down to a
  multiple of ``page_size`` and children are indexed by their first page;
* a partial match inside an edge splits the node at the (page-aligned) match
  point so that the matched part can be locked on its own;
* ``inc_lock_ref`` / ``dec_lock_ref`` pin the path from a node to the root while
  a running request uses it; pinned tokens count as *protected*, the others as
  *evictable*;
* ``evict(n)`` frees least-recently-used unpinned leaves until ``n`` tokens are
  released, moving up the tree as parents become leaves.

This is the pure-Python implementation; :mod:`mllm_b200.mem_cache.native`
offers the same tree in C++ for the scheduler's hot loop.
"""

from __future__ import annotations

import heapq
import itertools
import time
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from .base_prefix_cache import (
    BasePrefixCache, EvictResult, InsertResult, MatchResult, RadixKey, hash_token_ids,
)

_node_ids = itertools.count()
_EMPTY = np.empty((0,), dtype=np.int64)


class TreeNode:
    __slots__ = (
        "id", "children", "parent", "key", "value", "lock_ref", "last_access_time",
        "hit_count", "hash_value",
    )

    def __init__(self) -> None:
        self.id = next(_node_ids)
        self.children: Dict[object, "TreeNode"] = {}
        self.parent: Optional["TreeNode"] = None
        self.key: List[int] = []
        self.value: np.ndarray = _EMPTY
        self.lock_ref = 0
        self.last_access_time = time.monotonic()
        self.hit_count = 0
        self.hash_value: Optional[List[str]] = None

    @property
    def evicted(self) -> bool:
        return self.value is None

    def __lt__(self, other: "TreeNode") -> bool:
        return self.last_access_time < other.last_access_time


def _common_prefix_len(a: List[int], b: List[int], page: int) -> int:
    """Length of the common prefix of ``a`` and ``b``, rounded down to pages."""
    n = min(len(a), len(b))
    i = 0
    if page == 1:
        while i < n and a[i] == b[i]:
            i += 1
        return i
    while i + page <= n and a[i : i + page] == b[i : i + page]:
        i += page
    return i


class RadixCache(BasePrefixCache):
    def __init__(
        self,
        token_to_kv_pool_allocator=None,
        page_size: int = 1,
        on_evict: Optional[Callable[[np.ndarray], None]] = None,
        disable: bool = False,
    ) -> None:
        self.allocator = token_to_kv_pool_allocator
        self.page_size = int(page_size)
        self.on_evict = on_evict
        self.disable = disable
        self.reset()

    # -- bookkeeping -------------------------------------------------------
    def reset(self) -> None:
        self.root = TreeNode()
        self.root.lock_ref = 1  # never evicted
        self._evictable = 0
        self._protected = 0

    def evictable_size(self) -> int:
        return self._evictable

    def protected_size(self) -> int:
        return self._protected

    def total_size(self) -> int:
        total, stack = 0, [self.root]
        while stack:
            n = stack.pop()
            total += len(n.value)
            stack.extend(n.children.values())
        return total

    def _child_key(self, tokens: List[int], extra_key) -> object:
        head = tokens[0] if self.page_size == 1 else tuple(tokens[: self.page_size])
        return head if extra_key is None else (extra_key, head)

    def _aligned(self, n: int) -> int:
        return n - n % self.page_size

    # -- match -------------------------------------------------------------
    def match_prefix(self, key: RadixKey) -> MatchResult:
        tokens = key.token_ids[: self._aligned(len(key))]
        if self.disable or not tokens:
            return MatchResult(indices=_EMPTY, last_node=self.root, prefix_len=0)
        now = time.monotonic()
        node, pos, parts = self.root, 0, []
        node.last_access_time = now
        while pos < len(tokens):
            child = node.children.get(self._child_key(tokens[pos:], key.extra_key))
            if child is None:
                break
            m = _common_prefix_len(child.key, tokens[pos:], self.page_size)
            if m < len(child.key):
                if m > 0:
                    # only the matched part of a partially matched edge counts as used
                    upper = self._split(child, m, key.extra_key)
                    upper.last_access_time = now
                    parts.append(upper.value)
                    node = upper
                    pos += m
                break
            child.last_access_time = now
            parts.append(child.value)
            node = child
            pos += m
        node.hit_count += 1
        indices = np.concatenate(parts) if parts else _EMPTY
        return MatchResult(indices=indices, last_node=node, prefix_len=len(indices))

    # -- insert ------------------------------------------------------------
    def insert(self, key: RadixKey, value=None, **kw) -> InsertResult:
        if self.disable:
            return InsertResult(prefix_len=0, last_node=self.root)
        n = self._aligned(len(key))
        tokens = key.token_ids[:n]
        if value is None:
            value = np.asarray(tokens, dtype=np.int64)
        else:
            value = _as_np(value)[:n]
        now = time.monotonic()
        node, pos = self.root, 0
        while pos < n:
            ck = self._child_key(tokens[pos:], key.extra_key)
            child = node.children.get(ck)
            if child is None:
                leaf = TreeNode()
                leaf.parent = node
                leaf.key = tokens[pos:]
                leaf.value = value[pos:].copy()
                leaf.last_access_time = now
                node.children[ck] = leaf
                self._evictable += len(leaf.value)
                return InsertResult(prefix_len=pos, last_node=leaf)
            m = _common_prefix_len(child.key, tokens[pos:], self.page_size)
            if m < len(child.key):
                child = self._split(child, m, key.extra_key)
            child.last_access_time = now
            node = child
            pos += m
        return InsertResult(prefix_len=n, last_node=node)

    def _split(self, child: TreeNode, at: int, extra_key) -> TreeNode:
        """Cut ``child``'s edge at ``at`` tokens; return the new upper node."""
        upper = TreeNode()
        parent = child.parent
        upper.parent = parent
        upper.key, child.key = child.key[:at], child.key[at:]
        upper.value, child.value = child.value[:at], child.value[at:]
        upper.lock_ref = child.lock_ref
        upper.last_access_time = child.last_access_time
        if child.hash_value is not None:
            pages = at // self.page_size
            upper.hash_value, child.hash_value = child.hash_value[:pages], child.hash_value[pages:]
        parent.children[self._child_key(upper.key, extra_key_of(parent, child, extra_key))] = upper
        upper.children[self._child_key(child.key, extra_key)] = child
        child.parent = upper
        return upper

    # -- lock --------------------------------------------------------------
    def inc_lock_ref(self, node: Optional[TreeNode]):
        if self.disable or node is None:
            return 0
        delta = 0
        while node is not None and node is not self.root:
            if node.lock_ref == 0:
                n = len(node.value)
                self._evictable -= n
                self._protected += n
                delta -= n
            node.lock_ref += 1
            node = node.parent
        return delta

    def dec_lock_ref(self, node: Optional[TreeNode], **kw):
        if self.disable or node is None:
            return 0
        delta = 0
        while node is not None and node is not self.root:
            if node.lock_ref == 1:
                n = len(node.value)
                self._evictable += n
                self._protected -= n
                delta += n
            node.lock_ref -= 1
            assert node.lock_ref >= 0, "dec_lock_ref without matching inc_lock_ref"
            node = node.parent
        return delta

    # -- evict -------------------------------------------------------------
    def evict(self, num_tokens: int, swa_num_tokens: int = 0) -> EvictResult:
        if self.disable or num_tokens <= 0:
            return EvictResult()
        heap = [n for n in self._leaves() if n.lock_ref == 0]
        heapq.heapify(heap)
        freed = 0
        while freed < num_tokens and heap:
            node = heapq.heappop(heap)
            if node is self.root or node.lock_ref > 0 or node.children:
                continue
            self._release(node.value)
            freed += len(node.value)
            self._evictable -= len(node.value)
            parent = node.parent
            for k, v in list(parent.children.items()):
                if v is node:
                    del parent.children[k]
                    break
            if parent is not self.root and not parent.children and parent.lock_ref == 0:
                heapq.heappush(heap, parent)
        return EvictResult(full_evicted=freed)

    def _release(self, slots: np.ndarray) -> None:
        if self.on_evict is not None:
            self.on_evict(slots)
        if self.allocator is not None:
            self.allocator.free(slots)

    def _leaves(self) -> List[TreeNode]:
        out, stack = [], [self.root]
        while stack:
            n = stack.pop()
            if not n.children and n is not self.root:
                out.append(n)
            stack.extend(n.children.values())
        return out

    # -- hashes / debug ------------------------------------------------------
    def compute_node_hash(self, node: TreeNode) -> List[str]:
        """Chained SHA-256 of each page on ``node``'s edge (parent's last hash is the seed)."""
        if node.hash_value is not None:
            return node.hash_value
        prior = None
        if node.parent is not None and node.parent is not self.root:
            ph = self.compute_node_hash(node.parent)
            prior = ph[-1] if ph else None
        out = []
        for i in range(0, len(node.key), self.page_size):
            prior = hash_token_ids(node.key[i : i + self.page_size], prior)
            out.append(prior)
        node.hash_value = out
        return out

    def pretty_print(self) -> None:
        def rec(n: TreeNode, depth: int) -> None:
            print(" " * depth + f"[{len(n.key)}] lock={n.lock_ref} head={n.key[:6]}")
            for c in n.children.values():
                rec(c, depth + 2)

        rec(self.root, 0)
        print(f"evictable={self._evictable} protected={self._protected}")


def extra_key_of(parent: TreeNode, child: TreeNode, default):
    """Namespace under which ``child`` is filed in ``parent`` (recovered from the dict key)."""
    for k, v in parent.children.items():
        if v is child:
            if isinstance(k, tuple) and len(k) == 2 and isinstance(k[0], str):
                return k[0]
            return None
    return default


def _as_np(value) -> np.ndarray:
    if isinstance(value, np.ndarray):
        return value.astype(np.int64, copy=False)
    try:
        import torch

        if isinstance(value, torch.Tensor):
            return value.detach().to("cpu", torch.int64).numpy()
    except ImportError:  # pragma: no cover
        pass
    return np.asarray(value, dtype=np.int64)

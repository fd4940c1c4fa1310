"""Prefix cache for models whose sliding-window layers keep their K/V in a separate pool.

The full-attention layers need the K/V of the whole prefix; the sliding-window layers only of the last
``window`` tokens.  Under memory pressure the window pool's share of an *inner* part of a cached prefix can
therefore be given back while the full-attention share stays: such a node becomes a *tombstone* (role of the
SWA tombstones of pymllm/mem_cache/radix_cache.py:47-90,285-349).  Rules:

* a prefix is reusable only if the ``window`` tokens at its end are free of tombstones (or the whole prefix is):
  ``match_prefix`` returns the longest such prefix;
* ``insert`` may revive a tombstone with the inserting request's own slots when that request still holds the
  window K/V of those tokens (``swa_evicted_seqlen`` says from where on it does): the tree then owns the new
  slots and frees the old full-attention ones;
* ``evict(num_tokens, swa_num_tokens)`` first drops unlocked leaves (both pools), then, if more window-pool
  room is wanted, turns the least recently used unlocked nodes into tombstones via the allocator's ``free_swa``;
* a lock protects the full-attention K/V up to the root and the window K/V of the nodes that cover the last
  ``window`` tokens of the locked path.

Slots are shared between the pools (slot ``i`` of the window pool belongs to the same token as slot ``i`` of the
full pool); the allocator is expected to offer ``free(indices)`` for both and ``free_swa(indices)`` for the
window share alone.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional

import numpy as np

from .base_prefix_cache import BasePrefixCache, EvictResult, InsertResult, MatchResult, RadixKey

_EMPTY = np.empty(0, dtype=np.int64)


class SWATreeNode:
    __slots__ = ("id", "key", "value", "children", "parent", "swa_tombstone", "lock", "swa_lock")
    _next_id = 0

    def __init__(self) -> None:
        SWATreeNode._next_id += 1
        self.id = SWATreeNode._next_id
        self.key: List[int] = []
        self.value: np.ndarray = _EMPTY
        self.children: Dict[Any, "SWATreeNode"] = {}
        self.parent: Optional["SWATreeNode"] = None
        self.swa_tombstone = False
        self.lock = 0
        self.swa_lock = 0


class SWARadixCache(BasePrefixCache):
    def __init__(self, token_to_kv_pool_allocator: Any = None, page_size: int = 1, sliding_window_size: int = 0,
                 on_node_evict: Optional[Callable[[int], None]] = None) -> None:
        if sliding_window_size <= 0:
            raise ValueError("sliding_window_size must be positive")
        self.pool = token_to_kv_pool_allocator
        self.on_node_evict = on_node_evict            # called with the node id when a node leaves the tree
        self.page_size = max(1, int(page_size))
        self.window = int(sliding_window_size)
        self.reset()

    # ------------------------------------------------------------------ bookkeeping
    def reset(self) -> None:
        self.root_node = SWATreeNode()
        self.root_node.lock = self.root_node.swa_lock = 1
        self.lru: "OrderedDict[int, SWATreeNode]" = OrderedDict()
        self._evictable = self._protected = 0
        self._swa_evictable = self._swa_protected = 0
        # one entry per live lock: the nodes whose window K/V that lock protects (a split adds the new upper half)
        self._swa_holds: Dict[int, List[List[SWATreeNode]]] = {}

    def evictable_size(self) -> int:
        return self._evictable

    def protected_size(self) -> int:
        return self._protected

    def swa_evictable_size(self) -> int:
        return self._swa_evictable

    def swa_protected_size(self) -> int:
        return self._swa_protected

    def total_size(self) -> int:
        total, stack = 0, [self.root_node]
        while stack:
            n = stack.pop()
            total += len(n.value)
            stack.extend(n.children.values())
        return total

    def _align(self, n: int) -> int:
        return n - n % self.page_size

    def _child_key(self, tokens: List[int], extra_key, at_root: bool):
        head = tokens[0] if self.page_size == 1 else tuple(tokens[: self.page_size])
        return (extra_key, head) if at_root else head

    def _common(self, a: List[int], b: List[int]) -> int:
        n, i = min(len(a), len(b)), 0
        while i < n and a[i] == b[i]:
            i += 1
        return self._align(i)

    def _touch(self, node: SWATreeNode) -> None:
        path = []
        while node is not self.root_node:
            path.append(node)
            node = node.parent
        for n in reversed(path):
            self.lru[n.id] = n
            self.lru.move_to_end(n.id)

    # ------------------------------------------------------------------ walk / split
    def _walk(self, tokens: List[int], extra_key, split: bool):
        node, path, used = self.root_node, [], 0
        while used < len(tokens):
            rest = tokens[used:]
            if len(rest) < self.page_size:
                break
            child = node.children.get(self._child_key(rest, extra_key, node is self.root_node))
            if child is None:
                break
            m = self._common(child.key, rest)
            if m == 0:
                break
            if m < len(child.key):
                if not split:
                    break
                child = self._split(child, m)
            path.append(child)
            used += m
            node = child
        return path, used

    def _split(self, child: SWATreeNode, m: int) -> SWATreeNode:
        parent = child.parent
        upper = SWATreeNode()
        upper.key, upper.value, upper.parent = child.key[:m], child.value[:m].copy(), parent
        upper.swa_tombstone, upper.lock, upper.swa_lock = child.swa_tombstone, child.lock, child.swa_lock
        for k, v in parent.children.items():
            if v is child:
                parent.children[k] = upper
                break
        child.key, child.value, child.parent = child.key[m:], child.value[m:].copy(), upper
        upper.children[self._child_key(child.key, None, False)] = child
        self.lru[upper.id] = upper
        if child.swa_lock:
            for holds in self._swa_holds.values():
                for nodes in holds:
                    if any(n is child for n in nodes):
                        nodes.append(upper)
        return upper

    # ------------------------------------------------------------------ match
    def _usable(self, path: List[SWATreeNode]) -> int:
        """Number of leading nodes of ``path`` that form a reusable prefix."""
        best, clean, tail = 0, True, 0            # tail: tombstone-free tokens at the end of the prefix so far
        for i, n in enumerate(path):
            if n.swa_tombstone:
                clean, tail = False, 0
            else:
                tail += len(n.value)
            if clean or tail >= self.window:
                best = i + 1
        return best

    def match_prefix(self, key: RadixKey) -> MatchResult:
        tokens = list(key.token_ids)[: self._align(len(key))]
        if not tokens:
            return MatchResult(indices=_EMPTY, last_node=self.root_node, prefix_len=0)
        path, _ = self._walk(tokens, key.extra_key, split=True)
        nodes = path[: self._usable(path)]
        if not nodes:
            return MatchResult(indices=_EMPTY, last_node=self.root_node, prefix_len=0)
        self._touch(nodes[-1])
        idx = np.concatenate([n.value for n in nodes])
        return MatchResult(indices=idx, last_node=nodes[-1], prefix_len=len(idx))

    # ------------------------------------------------------------------ insert
    def insert(self, key: RadixKey, value=None, *, prev_prefix_len: int = 0, swa_evicted_seqlen: int = 0, **kw) -> InsertResult:
        """``value``: slots of the key's tokens.  ``prev_prefix_len``: tokens the request took from the tree (its
        slots for them *are* the tree's).  ``swa_evicted_seqlen``: the request's own window K/V is intact from this
        position on.  Returns the number of tokens the tree already held, tombstones revived here not counted
        (their slots were adopted, the caller must not free them)."""
        n = self._align(len(key))
        tokens = list(key.token_ids)[:n]
        value = (np.asarray(tokens, dtype=np.int64) if value is None else np.asarray(value, dtype=np.int64))[:n]
        if n == 0:
            return InsertResult()
        path, used = self._walk(tokens, key.extra_key, split=True)
        held, pos = 0, 0
        for node in path:
            length = len(node.value)
            revive = node.swa_tombstone and pos >= max(prev_prefix_len, swa_evicted_seqlen) and node.lock == 0
            if revive:
                if self.pool is not None:
                    self.pool.free(node.value)                      # the full-attention share of the old slots
                node.value = value[pos:pos + length].copy()
                node.swa_tombstone = False
                self._swa_evictable += length
            else:
                held += length
            pos += length
        node = path[-1] if path else self.root_node
        if used < n:
            leaf = SWATreeNode()
            leaf.key, leaf.value, leaf.parent = tokens[used:], value[used:].copy(), node
            node.children[self._child_key(leaf.key, key.extra_key, node is self.root_node)] = leaf
            self._evictable += len(leaf.value)
            self._swa_evictable += len(leaf.value)
            node = leaf
        self._touch(node)
        return InsertResult(prefix_len=held, last_node=node, adopted=used - held)

    # ------------------------------------------------------------------ locks
    def _window_nodes(self, node: SWATreeNode) -> List[SWATreeNode]:
        out, need = [], self.window
        while node is not self.root_node and need > 0:
            out.append(node)
            need -= len(node.value)
            node = node.parent
        return out

    def inc_lock_ref(self, node: Optional[SWATreeNode]):
        if node is None or node is self.root_node:
            return None
        held = self._window_nodes(node)
        self._swa_holds.setdefault(node.id, []).append(held)
        for n in held:
            if not n.swa_tombstone and n.swa_lock == 0:
                self._swa_evictable -= len(n.value)
                self._swa_protected += len(n.value)
            n.swa_lock += 1
        cur = node
        while cur is not self.root_node:
            if cur.lock == 0:
                self._evictable -= len(cur.value)
                self._protected += len(cur.value)
            cur.lock += 1
            cur = cur.parent
        return None

    def dec_lock_ref(self, node: Optional[SWATreeNode], **kw) -> None:
        if node is None or node is self.root_node:
            return
        holds = self._swa_holds.get(node.id)
        if not holds:
            raise ValueError("dec_lock_ref without a matching inc_lock_ref")
        held = holds.pop()
        if not holds:
            del self._swa_holds[node.id]
        for n in held:
            n.swa_lock -= 1
            if not n.swa_tombstone and n.swa_lock == 0:
                self._swa_evictable += len(n.value)
                self._swa_protected -= len(n.value)
        cur = node
        while cur is not self.root_node:
            cur.lock -= 1
            if cur.lock == 0:
                self._evictable += len(cur.value)
                self._protected -= len(cur.value)
            cur = cur.parent

    # ------------------------------------------------------------------ eviction
    def _drop_leaf(self, node: SWATreeNode) -> int:
        n = len(node.value)
        if self.pool is not None and n:
            if node.swa_tombstone and hasattr(self.pool, "free_full"):
                self.pool.free_full(node.value)                     # its window share went back earlier
            else:
                self.pool.free(node.value)
        parent = node.parent
        for k, v in list(parent.children.items()):
            if v is node:
                del parent.children[k]
                break
        self.lru.pop(node.id, None)
        self._evictable -= n
        if not node.swa_tombstone:
            self._swa_evictable -= n
        node.parent = None
        if self.on_node_evict is not None:
            self.on_node_evict(node.id)
        return n

    def evict(self, num_tokens: int, swa_num_tokens: int = 0) -> EvictResult:
        full = swa = 0
        while full < num_tokens:
            leaf = next((n for n in self.lru.values() if not n.children and n.lock == 0 and n.swa_lock == 0), None)
            if leaf is None:
                break
            if not leaf.swa_tombstone:
                swa += len(leaf.value)
            full += self._drop_leaf(leaf)
        while swa < swa_num_tokens:
            # an inner node may lose its window share while a request still holds its full-attention share
            node = next((n for n in self.lru.values()
                         if not n.swa_tombstone and n.swa_lock == 0 and (n.children or n.lock == 0)), None)
            if node is None:
                break
            if not node.children:          # a leaf without window K/V is of no use: drop it altogether
                swa += len(node.value)
                full += self._drop_leaf(node)
                continue
            if self.pool is not None and hasattr(self.pool, "free_swa"):
                self.pool.free_swa(node.value)
            node.swa_tombstone = True
            self._swa_evictable -= len(node.value)
            swa += len(node.value)
        return EvictResult(full_evicted=full, swa_evicted=swa)

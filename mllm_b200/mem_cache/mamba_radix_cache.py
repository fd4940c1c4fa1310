"""Prefix cache for hybrid models (full attention + gated-delta-net / SSM layers).

A cached prefix of such a model is only reusable where the recurrent state at its end is known: the
KV of the attention layers can be shared token by token, the recurrent state cannot be rebuilt from
it.  The tree therefore carries two values per node — the KV slots of the node's tokens and,
optionally, one *snapshot row* of the state pool holding the recurrent + convolution state after the
node's last token — with independent lock counts and independent LRU orders
(role of pymllm/mem_cache/mamba_radix_cache.py:48,113,227-640).

Rules of this implementation:

* ``match_prefix`` walks as far as the tokens match but reports, as the usable prefix, only the path
  down to the deepest node that holds a snapshot; ``mamba_branching_seqlen`` is the longer,
  KV-only match when there is one (a snapshot at that length would make it usable).
* a split puts the snapshot on the lower half (it describes the end of the original node); the upper
  half is a *tombstone* (KV, no state) until some request inserts a snapshot exactly there.
* ``insert`` takes ownership of the snapshot row it is given: adopted by the node, or returned to the
  pool when the node already has one.
* a KV lock covers the path to the root (a child's KV is meaningless without its ancestors'); a state
  lock covers the node only.
* eviction first drops unlocked leaves in LRU order (KV and snapshot together), then, if more
  snapshot rows are wanted, takes snapshots from unlocked nodes in their own LRU order; a leaf that
  loses its snapshot is dropped as well, since nothing can resume from it.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Any, Callable, Dict, List, Optional

import numpy as np

from .base_prefix_cache import BasePrefixCache, EvictResult, InsertResult, MatchResult, RadixKey

_EMPTY = np.empty(0, dtype=np.int64)


class MambaTreeNode:
    __slots__ = ("id", "key", "value", "children", "parent", "state_slot", "kv_lock", "state_lock", "hit_count")
    _next_id = 0

    def __init__(self) -> None:
        MambaTreeNode._next_id += 1
        self.id = MambaTreeNode._next_id
        self.key: List[int] = []
        self.value: np.ndarray = _EMPTY
        self.children: Dict[Any, "MambaTreeNode"] = {}
        self.parent: Optional["MambaTreeNode"] = None
        self.state_slot: Optional[int] = None
        self.kv_lock = 0
        self.state_lock = 0
        self.hit_count = 0

    @property
    def mamba_tombstone(self) -> bool:
        return self.state_slot is None

    def is_leaf(self) -> bool:
        return not self.children


class LRUOrder:
    """Least-recently-used order over nodes (oldest first), O(1) touch / remove."""

    def __init__(self) -> None:
        self._d: "OrderedDict[int, MambaTreeNode]" = OrderedDict()

    def __len__(self) -> int:
        return len(self._d)

    def __contains__(self, node: MambaTreeNode) -> bool:
        return node.id in self._d

    def touch(self, node: MambaTreeNode) -> None:
        self._d[node.id] = node
        self._d.move_to_end(node.id)

    def remove(self, node: MambaTreeNode) -> None:
        self._d.pop(node.id, None)

    def oldest(self, ok: Callable[[MambaTreeNode], bool]) -> Optional[MambaTreeNode]:
        for node in self._d.values():
            if ok(node):
                return node
        return None


class MambaRadixCache(BasePrefixCache):
    def __init__(self, token_to_kv_pool_allocator: Any = None, page_size: int = 1, mamba_pool: Any = None,
                 on_node_evict: Optional[Callable[[int], None]] = None) -> None:
        self.pool = token_to_kv_pool_allocator
        self.page_size = max(1, int(page_size))
        self.mamba_pool = mamba_pool
        self.on_node_evict = on_node_evict
        self.reset()

    # ------------------------------------------------------------------ bookkeeping
    def reset(self) -> None:
        self.root_node = MambaTreeNode()
        self.root_node.kv_lock = 1
        self.root_node.state_lock = 1
        self.kv_lru = LRUOrder()
        self.state_lru = LRUOrder()
        self._kv_evictable = self._kv_protected = 0
        self._state_evictable = self._state_protected = 0

    def evictable_size(self) -> int:
        return self._kv_evictable

    def protected_size(self) -> int:
        return self._kv_protected

    def mamba_evictable_size(self) -> int:
        return self._state_evictable

    def mamba_protected_size(self) -> int:
        return self._state_protected

    def total_size(self) -> int:
        total, stack = 0, [self.root_node]
        while stack:
            n = stack.pop()
            total += len(n.value)
            stack.extend(n.children.values())
        return total

    def snapshot_count(self) -> int:
        return self._state_evictable + self._state_protected

    # ------------------------------------------------------------------ keys
    def _align(self, n: int) -> int:
        return n - n % self.page_size

    def _child_key(self, tokens: List[int], extra_key, at_root: bool):
        head = tokens[0] if self.page_size == 1 else tuple(tokens[: self.page_size])
        return (extra_key, head) if at_root else head

    def _common(self, a: List[int], b: List[int]) -> int:
        n = min(len(a), len(b))
        i = 0
        while i < n and a[i] == b[i]:
            i += 1
        return self._align(i)

    def _touch_path(self, node: MambaTreeNode) -> None:
        path = []
        while node is not self.root_node:
            path.append(node)
            node = node.parent
        for n in reversed(path):  # ancestors first: a child always ends up younger than its parents
            self.kv_lru.touch(n)
            if n.state_slot is not None:
                self.state_lru.touch(n)

    # ------------------------------------------------------------------ match
    def _walk(self, tokens: List[int], extra_key, split: bool):
        """Follows ``tokens`` from the root.  Returns (nodes fully covered by the tokens, tokens they
        cover, further tokens matched inside the next node).  With ``split`` a partly matched node is
        cut so that its matched half joins the path (and the third value is 0)."""
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
                    return path, used, m
                child = self._split(child, m)
            child.hit_count += 1
            path.append(child)
            used += m
            node = child
        return path, used, 0

    def match_prefix(self, key: RadixKey) -> MatchResult:
        """Never cuts a node: the upper half of a cut has no snapshot, so it could not end a usable
        prefix anyway."""
        tokens = list(key.token_ids)[: self._align(len(key))]
        if not tokens:
            return MatchResult(indices=_EMPTY, last_node=self.root_node, prefix_len=0)
        path, used, partial = self._walk(tokens, key.extra_key, split=False)
        kv_len = used + partial
        usable = 0
        for i, n in enumerate(path):
            if n.state_slot is not None:
                usable = i + 1
        if usable == 0:
            return MatchResult(indices=_EMPTY, last_node=self.root_node, prefix_len=0,
                               mamba_branching_seqlen=kv_len or None)
        nodes = path[:usable]
        self._touch_path(nodes[-1])
        idx = np.concatenate([n.value for n in nodes])
        return MatchResult(indices=idx, last_node=nodes[-1], prefix_len=len(idx),
                           mamba_branching_seqlen=kv_len if kv_len > len(idx) else None,
                           state_slot=nodes[-1].state_slot)

    # ------------------------------------------------------------------ insert
    def insert(self, key: RadixKey, value=None, *, mamba_value: Optional[int] = None, **kw) -> InsertResult:
        """``value``: KV slots of the key's tokens.  ``mamba_value``: a snapshot row holding the state
        after the key's last token; the tree owns it from here on."""
        n = self._align(len(key))
        tokens = list(key.token_ids)[:n]
        if value is None:
            value = np.asarray(tokens, dtype=np.int64)
        value = np.asarray(value, dtype=np.int64)[:n]
        if n == 0:
            self._give_back(mamba_value)
            return InsertResult()
        path, used, _ = self._walk(tokens, key.extra_key, split=True)
        node = path[-1] if path else self.root_node
        if used < n:
            leaf = MambaTreeNode()
            leaf.key, leaf.value, leaf.parent = tokens[used:], value[used:].copy(), node
            node.children[self._child_key(leaf.key, key.extra_key, node is self.root_node)] = leaf
            self._kv_evictable += len(leaf.value)
            node = leaf
        existed = node.state_slot is not None
        if mamba_value is not None:
            if existed:
                self._give_back(mamba_value)
            else:
                node.state_slot = int(mamba_value)
                if node.state_lock > 0:
                    self._state_protected += 1
                else:
                    self._state_evictable += 1
        self._touch_path(node)
        return InsertResult(prefix_len=used, last_node=node, mamba_exist=existed)

    def _split(self, child: MambaTreeNode, m: int) -> MambaTreeNode:
        """Cuts ``child`` after ``m`` tokens; returns the new upper node (a tombstone)."""
        parent = child.parent
        upper = MambaTreeNode()
        upper.key, upper.value, upper.parent = child.key[:m], child.value[:m].copy(), parent
        upper.kv_lock = child.kv_lock           # every lock below passes through the upper half too
        for k, v in parent.children.items():
            if v is child:
                parent.children[k] = upper
                break
        child.key, child.value, child.parent = child.key[m:], child.value[m:].copy(), upper
        upper.children[self._child_key(child.key, None, False)] = child
        self.kv_lru.touch(upper)                # an inner node: its place matters only once it is a leaf again
        return upper

    # ------------------------------------------------------------------ locks
    def inc_lock_ref(self, node: Optional[MambaTreeNode]):
        if node is None or node is self.root_node:
            return None
        if node.state_slot is not None and node.state_lock == 0:
            self._state_evictable -= 1
            self._state_protected += 1
        node.state_lock += 1
        cur = node
        while cur is not self.root_node:
            if cur.kv_lock == 0:
                self._kv_evictable -= len(cur.value)
                self._kv_protected += len(cur.value)
            cur.kv_lock += 1
            cur = cur.parent
        return None

    def dec_lock_ref(self, node: Optional[MambaTreeNode], **kw) -> None:
        if node is None or node is self.root_node:
            return
        node.state_lock -= 1
        if node.state_slot is not None and node.state_lock == 0:
            self._state_evictable += 1
            self._state_protected -= 1
        cur = node
        while cur is not self.root_node:
            cur.kv_lock -= 1
            if cur.kv_lock == 0:
                self._kv_evictable += len(cur.value)
                self._kv_protected -= len(cur.value)
            cur = cur.parent

    # ------------------------------------------------------------------ eviction
    def _give_back(self, slot: Optional[int]) -> None:
        if slot is not None and self.mamba_pool is not None:
            self.mamba_pool.free_track_slot(int(slot))

    def _drop_state(self, node: MambaTreeNode) -> int:
        if node.state_slot is None:
            return 0
        self._give_back(node.state_slot)
        node.state_slot = None
        self.state_lru.remove(node)
        if node.state_lock > 0:
            self._state_protected -= 1
        else:
            self._state_evictable -= 1
        return 1

    def _drop_leaf(self, node: MambaTreeNode) -> int:
        """Removes an unlocked leaf; returns the KV tokens freed."""
        n = len(node.value)
        if self.pool is not None and n:
            self.pool.free(node.value)
        parent = node.parent
        for k, v in list(parent.children.items()):
            if v is node:
                del parent.children[k]
                break
        self.kv_lru.remove(node)
        self._kv_evictable -= n
        if self.on_node_evict is not None:
            self.on_node_evict(node.id)
        node.parent = None
        return n

    @staticmethod
    def _leaf_ok(n: MambaTreeNode) -> bool:
        return n.is_leaf() and n.kv_lock == 0 and n.state_lock == 0

    def evict(self, num_tokens: int, swa_num_tokens: int = 0, *, mamba_num: int = 0) -> EvictResult:
        """Frees at least ``num_tokens`` KV slots (while unlocked leaves remain) and at least
        ``mamba_num`` snapshot rows (``swa_num_tokens`` is accepted as an alias of the latter)."""
        want_state = max(int(mamba_num), int(swa_num_tokens))
        kv_freed = state_freed = 0
        while kv_freed < num_tokens:
            leaf = self.kv_lru.oldest(self._leaf_ok)
            if leaf is None:
                break
            state_freed += self._drop_state(leaf)
            kv_freed += self._drop_leaf(leaf)
        while state_freed < want_state:
            node = self.state_lru.oldest(lambda n: n.state_lock == 0)
            if node is None:
                break
            state_freed += self._drop_state(node)
            # nothing can resume from a stateless leaf: drop it, and the stateless chain above it
            while node is not self.root_node and self._leaf_ok(node) and node.state_slot is None:
                parent = node.parent
                kv_freed += self._drop_leaf(node)
                node = parent
        return EvictResult(full_evicted=kv_freed, mamba_evicted=state_freed)

    def alloc_state_slot(self) -> Optional[int]:
        """A free snapshot row of the state pool, evicting the least recently used snapshot if none is free."""
        if self.mamba_pool is None:
            return None
        slot = self.mamba_pool.alloc_track_slot()
        if slot is None and self.evict(0, mamba_num=1).mamba_evicted:
            slot = self.mamba_pool.alloc_track_slot()
        return slot

    # ------------------------------------------------------------------ debugging
    def pretty_print(self) -> str:
        lines: List[str] = []

        def rec(n: MambaTreeNode, depth: int) -> None:
            for c in n.children.values():
                lines.append(f"{'  ' * depth}{len(c.key)} tok kv_lock={c.kv_lock} state={c.state_slot} "
                             f"state_lock={c.state_lock}")
                rec(c, depth + 1)

        rec(self.root_node, 0)
        return "\n".join(lines)

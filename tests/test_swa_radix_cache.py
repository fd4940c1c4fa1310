"""Prefix cache with sliding-window tombstones (behaviour of pymllm/mem_cache/radix_cache.py's SWA mode)."""
import numpy as np
import pytest

from mllm_b200.mem_cache import RadixKey, SWARadixCache


class TwoPools:
    """Records which slots went back to which pool."""

    def __init__(self):
        self.full, self.swa = [], []

    def free(self, idx):
        self.full += list(map(int, idx))
        self.swa += list(map(int, idx))

    def free_full(self, idx):
        self.full += list(map(int, idx))

    def free_swa(self, idx):
        self.swa += list(map(int, idx))


def tombstone_head(c, a, b):
    la, lb = c.match_prefix(RadixKey(a)).last_node, c.match_prefix(RadixKey(b)).last_node
    c.inc_lock_ref(la), c.inc_lock_ref(lb)
    assert c.evict(0, 6).swa_evicted == 6
    c.dec_lock_ref(la), c.dec_lock_ref(lb)


def build(window=4):
    pool = TwoPools()
    c = SWARadixCache(pool, page_size=1, sliding_window_size=window)
    a = list(range(1, 13))                   # 12 tokens
    c.insert(RadixKey(a), np.arange(100, 112))
    b = a[:6] + [50, 51, 52, 53, 54, 55]     # shares 6 tokens: splits the first node
    c.insert(RadixKey(b), np.concatenate([np.arange(100, 106), np.arange(200, 206)]))
    return c, pool, a, b


def test_window_must_be_positive():
    with pytest.raises(ValueError):
        SWARadixCache(None, sliding_window_size=0)


def test_tombstone_keeps_full_kv_and_limits_reuse():
    c, pool, a, b = build()
    assert c.evictable_size() == 18 and c.swa_evictable_size() == 18
    # two running requests hold both branches: full-attention K/V of the whole paths, window K/V of the tails only
    la, lb = c.match_prefix(RadixKey(a)).last_node, c.match_prefix(RadixKey(b)).last_node
    c.inc_lock_ref(la), c.inc_lock_ref(lb)
    assert c.protected_size() == 18 and c.swa_protected_size() == 12 and c.swa_evictable_size() == 6
    # window-pool room is wanted: the shared head (inner, not window-locked) becomes a tombstone
    r = c.evict(0, 6)
    assert r.full_evicted == 0 and r.swa_evicted == 6
    assert sorted(pool.swa) == list(range(100, 106)) and pool.full == []
    assert c.swa_evictable_size() == 0 and c.evict(0, 6).swa_evicted == 0
    c.dec_lock_ref(la), c.dec_lock_ref(lb)
    assert c.evictable_size() == 18 and c.swa_evictable_size() == 12
    # the whole of `a` is still reusable: its last 6 tokens (>= window) are intact
    m = c.match_prefix(RadixKey(a))
    assert m.prefix_len == 12 and list(m.indices) == list(range(100, 112))
    # but a prefix ending inside or right after the tombstone is not: fewer than `window` intact tokens at its end
    assert c.match_prefix(RadixKey(a[:6] + [99])).prefix_len == 0
    assert c.match_prefix(RadixKey(a[:8] + [99])).prefix_len == 0          # 2 intact tokens < window
    assert c.match_prefix(RadixKey(a[:10] + [99])).prefix_len == 10        # 4 intact tokens == window


def test_insert_revives_tombstone_with_own_slots():
    c, pool, a, b = build()
    tombstone_head(c, a, b)
    # a request that recomputed everything (no reuse, window K/V intact from 0) hands in its own slots
    new = np.arange(300, 307)
    r = c.insert(RadixKey(a[:6] + [77]), new, prev_prefix_len=0, swa_evicted_seqlen=0)
    assert r.prefix_len == 0 and r.adopted == 6
    assert sorted(pool.full) == list(range(100, 106))                      # old full-attention slots went back
    m = c.match_prefix(RadixKey(a[:6] + [77]))
    assert m.prefix_len == 7 and list(m.indices) == list(range(300, 307))
    assert c.swa_evictable_size() == c.evictable_size() == 19
    # the old children now hang under the revived node with its new slots
    assert list(c.match_prefix(RadixKey(a)).indices) == list(range(300, 306)) + list(range(106, 112))


def test_insert_does_not_revive_without_window_kv():
    c, pool, a, b = build()
    tombstone_head(c, a, b)
    # the request's own window K/V of the first 6 tokens is gone (evicted up to position 8): nothing to adopt
    r = c.insert(RadixKey(a[:6] + [77]), np.arange(300, 307), swa_evicted_seqlen=8)
    assert r.prefix_len == 6 and r.adopted == 0 and pool.full == []
    assert c.match_prefix(RadixKey(a[:6] + [77, 78])).prefix_len == 0      # one intact token after the tombstone


def test_locks_protect_window_and_path():
    c, pool, a, b = build(window=4)
    m = c.match_prefix(RadixKey(a))
    c.inc_lock_ref(m.last_node)
    assert c.protected_size() == 12 and c.evictable_size() == 6
    assert c.swa_protected_size() == 6                # only the node covering the last 4 tokens is window-locked
    r = c.evict(100)
    # the unlocked branch of `b` goes (leaf, both pools); the locked path stays whole
    assert r.full_evicted == 6 and sorted(pool.full) == list(range(200, 206))
    assert c.match_prefix(RadixKey(a)).prefix_len == 12
    c.dec_lock_ref(m.last_node)
    assert c.protected_size() == 0 and c.swa_protected_size() == 0
    assert c.evictable_size() == 12 and c.swa_evictable_size() == 12
    r = c.evict(100)
    assert r.full_evicted == 12 and c.total_size() == 0
    assert sorted(pool.full) == sorted(pool.swa) == list(range(100, 112)) + list(range(200, 206))


def test_tombstoned_leaf_frees_only_full_share():
    gone = []
    c, pool, a, b = build()
    c.on_node_evict = gone.append
    tombstone_head(c, a, b)                           # shared head -> tombstone
    c.evict(12)                                       # both leaves go
    r = c.evict(6)                                    # the tombstone is a leaf now: only its full share is left
    assert r.full_evicted == 6 and r.swa_evicted == 0
    assert sorted(pool.swa) == sorted(pool.full) and len(pool.swa) == 18   # every slot returned exactly once per pool
    assert c.total_size() == 0 and c.evictable_size() == 0 and c.swa_evictable_size() == 0
    assert len(gone) == 3


def test_paged_keys_and_namespaces():
    c = SWARadixCache(TwoPools(), page_size=2, sliding_window_size=2)
    c.insert(RadixKey([1, 2, 3, 4, 5], extra_key="x"), np.arange(5))
    assert c.match_prefix(RadixKey([1, 2, 3, 4, 5], extra_key="x")).prefix_len == 4
    assert c.match_prefix(RadixKey([1, 2, 3, 4], extra_key="y")).prefix_len == 0
    assert c.match_prefix(RadixKey([1, 2, 3, 9], extra_key="x")).prefix_len == 2


def test_split_of_a_locked_node_keeps_lock_accounting():
    pool = TwoPools()
    c = SWARadixCache(pool, page_size=1, sliding_window_size=4)
    a = list(range(1, 13))
    c.insert(RadixKey(a), np.arange(100, 112))
    node = c.match_prefix(RadixKey(a)).last_node
    c.inc_lock_ref(node)
    assert c.swa_protected_size() == 12
    # another request shares 6 tokens: the locked node is split while the lock is held
    c.insert(RadixKey(a[:6] + [70, 71]), np.concatenate([np.arange(100, 106), np.arange(400, 402)]))
    assert c.swa_protected_size() == 12 and c.protected_size() == 12
    c.dec_lock_ref(node)
    assert c.swa_protected_size() == 0 and c.protected_size() == 0
    assert c.swa_evictable_size() == 14 and c.evictable_size() == 14
    assert c.evict(100).full_evicted == 14 and c.total_size() == 0
    with pytest.raises(ValueError):
        c.dec_lock_ref(node)

"""KV slot allocator, request table and radix prefix cache invariants."""
import numpy as np
import pytest
import torch

from mllm_b200.mem_cache import (ChunkCache, KVPool, RadixCache, RadixKey, ReqToTokenPool, TokenToKVPoolAllocator,
                                 hash_token_ids)


def test_allocator_token_granular():
    a = TokenToKVPoolAllocator(16, page_size=1)
    x = a.alloc_host(10)
    assert len(set(x.tolist())) == 10 and 0 not in x
    assert a.available_size() == 6 and a.alloc_host(7) is None
    a.free(x[:5])
    assert a.available_size() == 11
    y = a.alloc_host(11)
    assert y is not None and set(y.tolist()).isdisjoint(set(x[5:].tolist()))


def test_allocator_pages_and_groups():
    a = TokenToKVPoolAllocator(64, page_size=8)
    x = a.alloc_host(20)  # 3 pages
    assert a.available_size() == 64 - 24
    assert all(x[i] + 1 == x[i + 1] for i in range(7))  # slots of a page are consecutive
    a.free_group_begin()
    a.free(x[:8])
    a.free(x[8:])
    assert a.available_size() == 40
    a.free_group_end()
    assert a.available_size() == 64
    assert a.alloc(0).numel() == 0


def test_req_to_token_pool():
    p = ReqToTokenPool(4, 32, "cpu")
    s = p.alloc(3)
    assert p.alloc(2) is None
    p.write((s[0], slice(0, 4)), torch.arange(4))
    assert p.req_to_token[s[0], :4].tolist() == [0, 1, 2, 3]
    p.free(s)
    assert p.available_size() == 4


def test_kv_pool_layout_and_write():
    pool = KVPool(32, 2, 2, 128, torch.float32, "cpu", page_size=4)
    assert pool.k_buffer[0].shape == (36, 2, 128)
    k = torch.randn(3, 2, 128)
    v = torch.randn(3, 2, 128)
    pool.set_kv_buffer(1, torch.tensor([5, 9, 7]), k, v)
    assert torch.equal(pool.get_key_buffer(1)[9], k[1]) and torch.equal(pool.get_value_buffer(1)[7], v[2])
    assert pool.get_key_buffer(0).abs().sum() == 0


@pytest.mark.parametrize("page", [1, 4])
def test_radix_match_insert_split(page):
    alloc = TokenToKVPoolAllocator(256, page_size=page)
    rc = RadixCache(alloc, page_size=page)
    a = list(range(100, 116))
    va = alloc.alloc_host(16)
    assert rc.insert(RadixKey(a), va).prefix_len == 0
    assert rc.evictable_size() == 16
    # same prefix for 8 tokens, then diverges
    b = a[:8] + [7] * 8
    m = rc.match_prefix(RadixKey(b))
    assert m.prefix_len == 8 and np.array_equal(m.indices, va[:8])
    vb = alloc.alloc_host(8)
    r = rc.insert(RadixKey(b), np.concatenate([m.indices, vb]))
    assert r.prefix_len == 8 and rc.total_size() == 24
    # full re-match of both
    assert rc.match_prefix(RadixKey(a)).prefix_len == 16
    assert rc.match_prefix(RadixKey(b)).prefix_len == 16
    # unaligned tail is ignored
    assert rc.match_prefix(RadixKey(a[:8] + a[8:8 + page - 1] if page > 1 else a[:8])).prefix_len == 8


def test_radix_lock_and_lru_eviction():
    alloc = TokenToKVPoolAllocator(64, page_size=1)
    rc = RadixCache(alloc, page_size=1)
    seqs = [[i] * 4 + [50 + i] * 4 for i in range(4)]
    for s in seqs:
        rc.insert(RadixKey(s), alloc.alloc_host(8))
    assert alloc.available_size() == 32 and rc.evictable_size() == 32
    m = rc.match_prefix(RadixKey(seqs[0]))  # touch 0 (most recent) and pin it
    rc.inc_lock_ref(m.last_node)
    assert rc.protected_size() == 8 and rc.evictable_size() == 24
    res = rc.evict(100)
    assert res.full_evicted == 24 and alloc.available_size() == 56
    assert rc.match_prefix(RadixKey(seqs[0])).prefix_len == 8
    assert rc.match_prefix(RadixKey(seqs[1])).prefix_len == 0
    rc.dec_lock_ref(m.last_node)
    assert rc.evict(8).full_evicted == 8 and alloc.available_size() == 64


def test_radix_eviction_order_is_lru():
    alloc = TokenToKVPoolAllocator(64)
    rc = RadixCache(alloc)
    import time
    for i in range(3):
        rc.insert(RadixKey([i, i, i, i]), alloc.alloc_host(4))
        time.sleep(0.002)
    rc.match_prefix(RadixKey([0, 0, 0, 0]))  # refresh the oldest
    rc.evict(4)
    assert rc.match_prefix(RadixKey([1, 1, 1, 1])).prefix_len == 0
    assert rc.match_prefix(RadixKey([0, 0, 0, 0])).prefix_len == 4


def test_radix_extra_key_namespaces():
    rc = RadixCache(None)
    rc.insert(RadixKey([1, 2, 3], "img-a"), np.array([10, 11, 12]))
    assert rc.match_prefix(RadixKey([1, 2, 3], "img-b")).prefix_len == 0
    assert rc.match_prefix(RadixKey([1, 2, 3], "img-a")).prefix_len == 3
    assert rc.match_prefix(RadixKey([1, 2, 3])).prefix_len == 0


def test_page_hash_chain():
    h1 = hash_token_ids([1, 2, 3, 4])
    h2 = hash_token_ids([5, 6, 7, 8], h1)
    assert h2 != hash_token_ids([5, 6, 7, 8]) and len(h1) == 64
    rc = RadixCache(None, page_size=4)
    r = rc.insert(RadixKey(list(range(8))), np.arange(8))
    assert rc.compute_node_hash(r.last_node) == [hash_token_ids([0, 1, 2, 3]), hash_token_ids([4, 5, 6, 7], hash_token_ids([0, 1, 2, 3]))]


def test_chunk_cache_never_matches():
    cc = ChunkCache()
    assert cc.match_prefix(RadixKey([1, 2, 3])).prefix_len == 0
    assert cc.insert(RadixKey([1, 2, 3]), np.arange(3)).prefix_len == 0

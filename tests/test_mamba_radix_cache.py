"""State-aware prefix cache of hybrid models: tree rules, a randomized model check of its
bookkeeping, and an engine run where cached prefixes must not change any generated token."""

import random

import numpy as np
import pytest

from mllm_b200.mem_cache import MambaRadixCache, RadixKey


class FakeKV:
    def __init__(self, n):
        self.free_set = set(range(n))

    def alloc(self, n):
        out = [self.free_set.pop() for _ in range(n)]
        return np.asarray(out, dtype=np.int64)

    def free(self, idx):
        for i in np.asarray(idx).tolist():
            assert i not in self.free_set, "double free of a KV slot"
            self.free_set.add(i)


class FakeStates:
    """Snapshot rows 100..100+n-1."""

    def __init__(self, n):
        self.slots, self.track_slots = 100, n
        self.free_rows = list(range(100, 100 + n))

    def alloc_track_slot(self):
        return self.free_rows.pop() if self.free_rows else None

    def free_track_slot(self, s):
        assert 100 <= s < 100 + self.track_slots and s not in self.free_rows, "bad snapshot row free"
        self.free_rows.append(s)


def _cache(page=1, kv=1000, states=8):
    kvp, stp = FakeKV(kv), FakeStates(states)
    return MambaRadixCache(kvp, page, stp), kvp, stp


def test_usable_prefix_ends_at_a_snapshot():
    c, kv, st = _cache()
    a = list(range(10))
    r = c.insert(RadixKey(a), kv.alloc(10), mamba_value=st.alloc_track_slot())
    assert r.prefix_len == 0 and not r.mamba_exist
    m = c.match_prefix(RadixKey(a + [77, 78]))
    assert m.prefix_len == 10 and m.state_slot == r.last_node.state_slot and m.mamba_branching_seqlen is None
    # a shorter or diverging prompt shares KV with the node but there is no state at that point
    m = c.match_prefix(RadixKey(a[:6] + [50, 51]))
    assert m.prefix_len == 0 and m.mamba_branching_seqlen == 6 and m.last_node is c.root_node
    # inserting the diverging sequence cuts the node: upper half tombstone, lower half keeps the snapshot
    b = a[:6] + [50, 51]
    vb = np.concatenate([r.last_node.value[:6], kv.alloc(2)])
    rb = c.insert(RadixKey(b), vb, mamba_value=st.alloc_track_slot())
    assert rb.prefix_len == 6
    assert c.match_prefix(RadixKey(a)).prefix_len == 10
    assert c.match_prefix(RadixKey(b + [1])).prefix_len == 8
    assert c.match_prefix(RadixKey(a[:6])).prefix_len == 0          # tombstone
    # a snapshot inserted exactly at the cut makes it usable
    rc = c.insert(RadixKey(a[:6]), vb[:6], mamba_value=st.alloc_track_slot())
    assert rc.prefix_len == 6 and not rc.mamba_exist
    assert c.match_prefix(RadixKey(a[:6] + [99])).prefix_len == 6
    # a second snapshot for the same node goes back to the pool
    free_before = len(st.free_rows)
    rd = c.insert(RadixKey(a[:6]), vb[:6], mamba_value=st.alloc_track_slot())
    assert rd.mamba_exist and len(st.free_rows) == free_before
    assert c.snapshot_count() == 3 and c.total_size() == 12


def test_locks_and_two_phase_eviction():
    c, kv, st = _cache(states=3)
    seqs = [[1, 2, 3, 4], [1, 2, 3, 4, 5, 6], [9, 9, 9]]
    nodes = []
    for s in seqs:
        pre = c.match_prefix(RadixKey(s))
        val = np.concatenate([pre.indices, kv.alloc(len(s) - pre.prefix_len)])
        nodes.append(c.insert(RadixKey(s), val, mamba_value=st.alloc_track_slot()).last_node)
    assert c.evictable_size() == 9 and c.mamba_evictable_size() == 3 and not st.free_rows
    c.inc_lock_ref(nodes[1])                      # locks [1,2,3,4] (KV only) and its child (KV + state)
    assert c.protected_size() == 6 and c.mamba_protected_size() == 1
    # snapshot pressure: the oldest unlocked snapshot goes first ([1,2,3,4]: an inner node keeps its KV)
    slot = c.alloc_state_slot()
    assert slot is not None and nodes[0].state_slot is None and c.total_size() == 9
    st.free_track_slot(slot)
    # KV pressure: only the unlocked leaf can go, with its snapshot
    res = c.evict(100)
    assert res.full_evicted == 3 and res.mamba_evicted == 1 and c.total_size() == 6
    c.dec_lock_ref(nodes[1])
    assert c.protected_size() == 0 and c.evictable_size() == 6
    res = c.evict(100)
    assert res.full_evicted == 6 and c.total_size() == 0 and len(st.free_rows) == 3 and len(kv.free_set) == 1000


def test_leaf_that_loses_its_snapshot_is_dropped():
    c, kv, st = _cache(states=2)
    c.insert(RadixKey([1, 2, 3]), kv.alloc(3), mamba_value=st.alloc_track_slot())
    c.insert(RadixKey([4, 5]), kv.alloc(2), mamba_value=st.alloc_track_slot())
    assert c.alloc_state_slot() is not None       # takes the snapshot of [1,2,3], which then has no use
    assert c.total_size() == 2 and c.match_prefix(RadixKey([1, 2, 3, 4])).prefix_len == 0


@pytest.mark.parametrize("page", [1, 4])
def test_randomized_bookkeeping(page):
    rng = random.Random(1234 + page)
    c, kv, st = _cache(page=page, kv=4000, states=6)
    locked = []
    for step in range(600):
        op = rng.random()
        if op < 0.55:
            n = rng.randrange(1, 40)
            seq = [rng.randrange(3) for _ in range(n)]          # tiny alphabet: lots of shared prefixes
            n_al = n - n % page
            m = c.match_prefix(RadixKey(seq))
            assert m.prefix_len % page == 0 and m.prefix_len <= n_al
            if m.prefix_len:
                assert m.state_slot is not None and m.last_node.state_slot == m.state_slot
            if n_al > m.prefix_len:
                snap = c.alloc_state_slot()
                if snap is None:
                    continue
                fresh = kv.alloc(n_al - m.prefix_len)
                r = c.insert(RadixKey(seq[:n_al]), np.concatenate([m.indices, fresh]), mamba_value=snap)
                # tokens the tree already held beyond the usable prefix: our slots for them are duplicates
                if r.prefix_len > m.prefix_len:
                    kv.free(fresh[: r.prefix_len - m.prefix_len])
                if rng.random() < 0.3:
                    c.inc_lock_ref(r.last_node)
                    locked.append(r.last_node)
        elif op < 0.75 and locked:
            c.dec_lock_ref(locked.pop(rng.randrange(len(locked))))
        else:
            c.evict(rng.randrange(0, 30), mamba_num=rng.randrange(0, 2))
        # ---- invariants ----
        total, snaps, prot, sprot = 0, 0, 0, 0
        stack = [c.root_node]
        while stack:
            nd = stack.pop()
            for ch in nd.children.values():
                assert ch.parent is nd and len(ch.key) == len(ch.value) and len(ch.key) % page == 0 and len(ch.key) > 0
                assert ch.kv_lock >= sum(g.kv_lock for g in ch.children.values())
                total += len(ch.value)
                prot += len(ch.value) if ch.kv_lock else 0
                snaps += ch.state_slot is not None
                sprot += ch.state_slot is not None and ch.state_lock > 0
                stack.append(ch)
        assert total == c.total_size() == c.evictable_size() + c.protected_size()
        assert prot == c.protected_size()
        assert snaps == c.snapshot_count() == st.track_slots - len(st.free_rows)
        assert sprot == c.mamba_protected_size()
        assert total + len(kv.free_set) == 4000
    for nd in locked:
        c.dec_lock_ref(nd)
    c.evict(10 ** 9, mamba_num=10 ** 9)
    assert c.total_size() == 0 and len(kv.free_set) == 4000 and len(st.free_rows) == st.track_slots


def test_hybrid_engine_with_state_cache_reproduces_uncached_tokens():
    """Qwen3.5-tiny through the scheduler: multi-turn style prompts (each extends an earlier prompt plus
    its answer) give the same tokens with the state-aware cache as with no prefix reuse, and the cache
    really serves prefixes."""
    from mllm_b200.configs import ServerConfig
    from mllm_b200.engine.launch import Engine

    def run(enable, slots=12):
        cfg = ServerConfig(model_path="preset:qwen3.5-tiny", dtype="float32", max_running_requests=4,
                           max_total_tokens=2048, context_length=256, log_level="warning",
                           enable_mamba_cache=enable, mamba_cache_slots=slots if enable else None)
        eng = Engine(cfg, mode="inproc", device="cpu").launch()
        try:
            outs, hits = [], []
            base = [5, 9, 2, 7, 7, 3, 1, 8, 4, 6, 2, 2]
            history = list(base)
            for turn in range(4):
                r = eng.generate(input_ids=list(history), sampling_params={"max_new_tokens": 6, "temperature": 0.0})
                outs.append(r["output_ids"])
                hits.append(r["meta_info"]["cached_tokens"])
                history = history + r["output_ids"] + [11 + turn, 3]
            r = eng.generate(input_ids=base + [40, 41], sampling_params={"max_new_tokens": 4, "temperature": 0.0})
            outs.append(r["output_ids"])
            hits.append(r["meta_info"]["cached_tokens"])
            mrp = eng.scheduler.mrp
            return outs, hits, type(mrp.prefix_cache).__name__
        finally:
            eng.shutdown()

    plain, hits0, kind0 = run(False)
    cached, hits1, kind1 = run(True)
    assert kind0 == "ChunkCache" and kind1 == "MambaRadixCache"
    assert hits0 == [0] * 5
    assert cached == plain
    assert hits1[0] == 0 and all(h > 0 for h in hits1[1:4])      # each turn resumes from the previous one
    assert hits1[4] == len([5, 9, 2, 7, 7, 3, 1, 8, 4, 6, 2, 2])  # the first prompt's own snapshot
    # two snapshot rows only: snapshots are evicted all the time, tokens must not change
    tight, _, _ = run(True, slots=2)
    assert tight == plain


def test_hybrid_model_batched_chunked_mixed_equals_one_at_a_time():
    """Five requests with shared prefixes submitted together to a hybrid model with small prefill chunks (so
    prefill chunks of some requests ride in the same pass as decode steps of others) and the state-aware
    cache on: every request gets the tokens it gets alone, without any cache."""
    from mllm_b200.configs import ServerConfig
    from mllm_b200.engine.io_struct import TokenizedGenerateReqInput
    from mllm_b200.orchestrator.scheduler_process import build_scheduler

    base = [5, 9, 2, 7, 7, 3, 1, 8, 4, 6, 2, 2, 9, 9, 1]
    prompts = [base, base + [40, 41, 42], base[:9] + [60, 61], [70, 71, 72, 73], base + [40, 41, 42, 43, 44, 45, 46]]

    def cfg(**kw):
        return ServerConfig(model_path="preset:qwen3.5-tiny", dtype="float32", max_total_tokens=2048, context_length=256,
                            log_level="warning", **kw)

    def drain(sched):
        done = {}
        for _ in range(800):
            out = sched.step()
            if out is not None:
                for i, rid in enumerate(out.rids):
                    if out.finished_reasons[i] is not None:
                        done[rid] = out.output_ids[i]
            if not sched.has_work():
                break
        return done

    def req(rid, ids):
        return TokenizedGenerateReqInput(rid=rid, input_ids=list(ids), sampling_params=dict(max_new_tokens=7, temperature=0.0))

    alone = {}
    for i, p in enumerate(prompts):
        s = build_scheduler(cfg(max_running_requests=1, disable_radix_cache=True), device="cpu")
        s.add_request(req(f"r{i}", p))
        alone.update(drain(s))
    sched = build_scheduler(cfg(max_running_requests=4, chunked_prefill_size=8, enable_mamba_cache=True, mamba_cache_slots=8),
                            device="cpu")
    for i, p in enumerate(prompts[:3]):
        sched.add_request(req(f"r{i}", p))
    for _ in range(3):
        sched.step()
    for i, p in enumerate(prompts[3:], start=3):
        sched.add_request(req(f"r{i}", p))
    together = drain(sched)
    assert together == alone
    assert sched.stats.num_mixed_batches > 0
    sched._sweep_finished()
    mrp = sched.mrp
    assert mrp.prefix_cache.protected_size() == 0 and mrp.prefix_cache.mamba_protected_size() == 0

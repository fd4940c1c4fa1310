"""Host-native C++ components against their Python twins: randomised differential tests of the radix
tree and the slot allocator, byte-level fixtures of the .mllm reader/writer, GGUF block expansion."""
import random
import struct

import numpy as np
import pytest
import torch

from mllm_b200.io.mllm_file import MllmFileReader, iter_mllm_tensors, write_mllm, write_mllm_v1
from mllm_b200.mem_cache import RadixCache, RadixKey, TokenToKVPoolAllocator
from mllm_b200.mem_cache.native import NativeRadixCache, NativeTokenToKVPoolAllocator, host_ext


@pytest.mark.parametrize("page", [1, 4])
def test_radix_tree_matches_python(page, monkeypatch):
    # a logical clock on the Python side too, so both trees evict in exactly the same order
    import itertools

    from mllm_b200.mem_cache import radix_cache as rc_mod

    ticks = itertools.count(1)
    monkeypatch.setattr(rc_mod.time, "monotonic", lambda: float(next(ticks)))
    rng = random.Random(page)
    py_alloc, nat_alloc = TokenToKVPoolAllocator(4096, page), TokenToKVPoolAllocator(4096, page)
    py, nat = RadixCache(py_alloc, page), NativeRadixCache(nat_alloc, page)
    locked = []
    for step in range(400):
        op = rng.random()
        base = [rng.randrange(3) for _ in range(rng.randrange(1, 6) * page)]
        toks = base + [rng.randrange(50) for _ in range(rng.randrange(0, 5) * page)]
        extra = rng.choice([None, None, "lora-a"])
        key = RadixKey(toks, extra)
        if op < 0.45:
            n = len(toks) - len(toks) % page
            slots = py_alloc.alloc_host(n)
            slots2 = nat_alloc.alloc_host(n)
            if slots is None:
                continue
            a, b = py.insert(key, slots), nat.insert(key, slots2)
            assert a.prefix_len == b.prefix_len
            # duplicates (already cached) go back to the pool, as the scheduler does
            py_alloc.free(slots[: a.prefix_len])
            nat_alloc.free(slots2[: b.prefix_len])
        elif op < 0.8:
            a, b = py.match_prefix(key), nat.match_prefix(key)
            assert a.prefix_len == b.prefix_len
            if rng.random() < 0.3 and a.prefix_len:
                py.inc_lock_ref(a.last_node)
                nat.inc_lock_ref(b.last_node)
                locked.append((a.last_node, b.last_node))
        elif op < 0.9 and locked:
            a, b = locked.pop(rng.randrange(len(locked)))
            py.dec_lock_ref(a)
            nat.dec_lock_ref(b)
        else:
            n = rng.randrange(1, 20) * page
            a, b = py.evict(n), nat.evict(n)
            assert (a.full_evicted >= n or py.evictable_size() == 0) and (b.full_evicted >= n or nat.evictable_size() == 0)
        assert py.protected_size() == nat.protected_size(), step
        assert py.protected_size() + py.evictable_size() == py.total_size()
        assert nat.protected_size() + nat.evictable_size() == nat.total_size()
        # every cached token is backed by a slot that is not free: sizes + free slots add up
        assert nat.total_size() + nat_alloc.available_size() == 4096 // page * page
    for a, b in locked:
        py.dec_lock_ref(a)
        nat.dec_lock_ref(b)
    nat.evict(10 ** 9)
    assert nat.total_size() == 0 and nat_alloc.available_size() == 4096 // page * page


def test_native_lru_order_and_lock_protection():
    nat = NativeRadixCache(None, 1)
    nat.insert(RadixKey([1, 2, 3]), np.array([10, 11, 12]))
    nat.insert(RadixKey([1, 2, 4]), np.array([10, 11, 13]))
    nat.insert(RadixKey([7, 8]), np.array([20, 21]))
    m = nat.match_prefix(RadixKey([1, 2, 3]))          # touches [1,2] and [3]
    assert m.indices.tolist() == [10, 11, 12]
    nat.inc_lock_ref(m.last_node)
    assert nat.protected_size() == 3 and nat.evictable_size() == 3
    freed = []
    nat.on_evict = lambda s: freed.extend(s.tolist())
    nat.evict(100)
    assert sorted(freed) == [13, 20, 21]              # the locked path survives
    nat.dec_lock_ref(m.last_node)
    nat.evict(100)
    assert sorted(freed) == [10, 11, 12, 13, 20, 21] and nat.total_size() == 0


def test_native_namespaces_with_any_hash_value():
    """Namespaces (image hashes, adapter ids) hash to unsigned 64-bit values; the tree's key is signed: both
    halves of the range must work and stay distinct."""
    nat = NativeRadixCache(None, 1)
    for i in range(20):                                 # "img2", "img3", ... hash into the upper half
        nat.insert(RadixKey([1, 2, 3], extra_key=f"img{i}"), np.array([100 * i, 100 * i + 1, 100 * i + 2]))
    for i in range(20):
        assert nat.match_prefix(RadixKey([1, 2, 3, 4], extra_key=f"img{i}")).indices.tolist() == [100 * i, 100 * i + 1, 100 * i + 2]
    assert nat.match_prefix(RadixKey([1, 2, 3])).prefix_len == 0 and nat.total_size() == 60


@pytest.mark.parametrize("page", [1, 8])
def test_allocator_matches_python(page):
    rng = random.Random(0)
    py, nat = TokenToKVPoolAllocator(1024, page), NativeTokenToKVPoolAllocator(1024, page)
    held = []
    for _ in range(300):
        if rng.random() < 0.6 or not held:
            n = rng.randrange(1, 40)
            a, b = py.alloc_host(n), nat.alloc_host(n)
            assert (a is None) == (b is None)
            if a is not None:
                assert len(a) == len(b) and len(set(b.tolist())) == len(b) and min(b) >= page
                held.append((a, b))
        else:
            a, b = held.pop(rng.randrange(len(held)))
            py.free(a)
            nat.free(b)
        assert py.available_size() == nat.available_size()
    live = np.concatenate([b for _, b in held]) if held else np.empty(0, dtype=np.int64)
    assert len(set(live.tolist())) == len(live)


def test_mllm_v2_roundtrip_and_layout(tmp_path):
    torch.manual_seed(0)
    tensors = [("model.embed_tokens.weight", torch.randn(7, 5).to(torch.bfloat16)),
               ("model.layers.0.self_attn.q_proj.weight", torch.randn(4, 6)),
               ("w.int8", torch.randint(-128, 127, (3, 9), dtype=torch.int8)),
               ("scale.f16", torch.randn(11).to(torch.float16)), ("idx", torch.arange(5, dtype=torch.int32))]
    path = str(tmp_path / "m.mllm")
    write_mllm(path, tensors, model_name="tiny")
    raw = open(path, "rb").read()
    magic, ver, name, n, desc = struct.unpack_from("<II512sIQ", raw, 0)
    assert (magic, ver, n, desc) == (0x519A, 2, 5, 532) and name.rstrip(b"\0") == b"tiny"
    pid, dt, size, off, rank, *rest = struct.unpack_from("<IIQQQ16i256s", raw, 532)
    assert (pid, dt, size, rank, rest[:2]) == (0, 128, 70, 2, [7, 5]) and rest[16].rstrip(b"\0") == b"model.embed_tokens.weight"
    assert off % 64 == 0 and raw[off:off + 70] == tensors[0][1].view(torch.uint8).numpy().tobytes()
    r = MllmFileReader(path)
    assert r.version == 2 and r.model_name == "tiny" and r.names() == [n for n, _ in tensors]
    for (name, want), (name2, got) in zip(tensors, iter_mllm_tensors(path)):
        assert name == name2 and got.dtype == want.dtype and torch.equal(got, want)


def test_mllm_v1_read(tmp_path):
    tensors = [("a.weight", torch.randn(3, 4)), ("b.bias", torch.randn(6).to(torch.float16))]
    path = str(tmp_path / "old.mllm")
    write_mllm_v1(path, tensors)
    r = MllmFileReader(path)
    assert r.version == 1 and r.names() == ["a.weight", "b.bias"]
    got = dict(iter_mllm_tensors(path))
    assert torch.equal(got["a.weight"], tensors[0][1].reshape(-1))       # V1 stores no shapes
    assert torch.equal(got["b.bias"], tensors[1][1])


def test_mllm_rejects_garbage(tmp_path):
    p = tmp_path / "bad.mllm"
    p.write_bytes(b"\x01\x02\x03\x04" * 10)
    with pytest.raises(RuntimeError):
        MllmFileReader(str(p))


def _q4_0_blocks(x: np.ndarray) -> bytes:
    out = b""
    for blk in x.reshape(-1, 32):
        amax_idx = np.abs(blk).argmax()
        d = blk[amax_idx] / -8.0 if blk[amax_idx] != 0 else 1.0
        d16 = np.float16(d)
        q = np.clip(np.round(blk / np.float32(d16)) + 8, 0, 15).astype(np.uint8)
        out += d16.tobytes() + (q[:16] | (q[16:] << 4)).astype(np.uint8).tobytes()
    return out


def test_gguf_q4_0_and_q8_0_expansion():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(64 * 32).astype(np.float32)
    raw = np.frombuffer(_q4_0_blocks(x), dtype=np.uint8)
    got = host_ext().gguf_dequantize(2, raw, 2)
    # independent restatement of the block layout: value j = ((nibble) - 8) * d, low nibbles first
    want = []
    for b in raw.reshape(-1, 18):
        d = np.frombuffer(b[:2].tobytes(), dtype=np.float16)[0].astype(np.float32)
        qs = b[2:]
        want += [((qs & 15).astype(np.int32) - 8) * d, ((qs >> 4).astype(np.int32) - 8) * d]
    np.testing.assert_array_equal(got, np.concatenate(want).astype(np.float32))
    assert np.abs(got - x).max() < 0.6
    # Q8_0
    blocks = b""
    xs = x.reshape(-1, 32)
    for blk in xs:
        d16 = np.float16(np.abs(blk).max() / 127.0)
        blocks += d16.tobytes() + np.clip(np.round(blk / np.float32(d16)), -127, 127).astype(np.int8).tobytes()
    got8 = host_ext().gguf_dequantize(8, np.frombuffer(blocks, dtype=np.uint8), 1)
    assert np.abs(got8 - x).max() < 0.05


def test_gguf_k_quants_known_blocks():
    """Q4_K / Q6_K super-blocks built by hand from the published layout; expansion must give back
    d * scale * q - dmin * min (Q4_K) and d * scale * (q - 32) (Q6_K)."""
    # Q4_K: all 8 sub-block scales = 2, mins = 1 (6-bit fields), nibbles = position mod 16
    d, dmin = np.float16(0.5), np.float16(0.25)
    scales = bytearray(12)
    for j in range(4):
        scales[j] = 2
        scales[j + 4] = 1
    for j in range(4, 8):
        scales[j + 4] = (2 & 0xF) | ((1 & 0xF) << 4)   # high two bits of both fields are zero
    qs = bytearray(128)
    vals = np.arange(256) % 16
    for grp in range(4):
        lo, hi = vals[grp * 64: grp * 64 + 32], vals[grp * 64 + 32: grp * 64 + 64]
        for l in range(32):
            qs[grp * 32 + l] = int(lo[l]) | (int(hi[l]) << 4)
    blk = d.tobytes() + dmin.tobytes() + bytes(scales) + bytes(qs)
    assert len(blk) == 144
    got = host_ext().gguf_dequantize(12, np.frombuffer(blk, dtype=np.uint8), 1)
    np.testing.assert_allclose(got, 0.5 * 2 * vals - 0.25 * 1, rtol=0, atol=1e-6)
    # Q6_K: scales = 3, q = 40 everywhere (low nibble 8, high bits 2) -> d * 3 * (40 - 32)
    ql = bytes([8 | (8 << 4)] * 128)
    qh = bytes([2 | (2 << 2) | (2 << 4) | (2 << 6)] * 64)
    sc = bytes([3] * 16)
    blk6 = ql + qh + sc + np.float16(0.125).tobytes()
    assert len(blk6) == 210
    got6 = host_ext().gguf_dequantize(14, np.frombuffer(blk6, dtype=np.uint8), 1)
    np.testing.assert_allclose(got6, np.full(256, 0.125 * 3 * 8, dtype=np.float32))


def test_convert_roundtrip_and_model_load(tmp_path):
    """safetensors -> .mllm -> model: a tiny Qwen3 loaded from the .mllm file gives the logits of the same
    weights loaded from safetensors (the loader path the server takes for ``*.mllm`` checkpoints)."""
    from safetensors.torch import save_file

    from mllm_b200.configs import ServerConfig
    from mllm_b200.executor import ModelRunner
    from mllm_b200.io.convert import main as convert_main
    from mllm_b200.models.presets import get_preset, preset_to_config_json

    import json

    cfg = get_preset("qwen3-tiny")
    sc = ServerConfig(model_path="preset:qwen3-tiny", dtype="float32", max_running_requests=2, max_total_tokens=256)
    src = ModelRunner(sc, hf_config=cfg, device="cpu")
    src.initialize()
    hf_names = {}
    for name, p in src.model.named_parameters():
        hf_names[name] = p.detach().clone()
    # un-fuse into HF names so both loaders exercise their stacking logic
    sd = {}
    for name, t in hf_names.items():
        if ".qkv_proj." in name:
            q = cfg.num_attention_heads * cfg.head_dim
            kv = cfg.num_key_value_heads * cfg.head_dim
            sd[name.replace("qkv_proj", "q_proj")] = t[:q].clone()
            sd[name.replace("qkv_proj", "k_proj")] = t[q:q + kv].clone()
            sd[name.replace("qkv_proj", "v_proj")] = t[q + kv:].clone()
        elif ".gate_up_proj." in name:
            from mllm_b200 import ops

            v = t.reshape(-1, 2, ops.SWIGLU_BLOCK, t.shape[1]) if t.shape[0] % (2 * ops.SWIGLU_BLOCK) == 0 else None
            g = v[:, 0].reshape(-1, t.shape[1]) if v is not None else t[: t.shape[0] // 2]
            u = v[:, 1].reshape(-1, t.shape[1]) if v is not None else t[t.shape[0] // 2:]
            sd[name.replace("gate_up_proj", "gate_proj")] = g.clone()
            sd[name.replace("gate_up_proj", "up_proj")] = u.clone()
        else:
            sd[name] = t
    st_dir, ml_dir = tmp_path / "st", tmp_path / "ml"
    st_dir.mkdir()
    ml_dir.mkdir()
    save_file(sd, str(st_dir / "model.safetensors"))
    for d in (st_dir, ml_dir):
        (d / "config.json").write_text(json.dumps(preset_to_config_json("qwen3-tiny")))
    convert_main(["--input", str(st_dir), "--output", str(ml_dir / "model.mllm"), "--model-name", "tiny"])
    convert_main(["--input", str(ml_dir / "model.mllm"), "--output", str(tmp_path / "x"), "--list"])

    def logits(path):
        mr = ModelRunner(ServerConfig(model_path=str(path), dtype="float32", max_running_requests=2, max_total_tokens=256),
                         device="cpu")
        mr.initialize()
        ids = torch.arange(5, 14)
        slots = mr.req_to_token_pool.alloc(1)
        loc = mr.token_to_kv_pool_allocator.alloc(9)
        mr.req_to_token_pool.req_to_token[slots[0], :9] = loc.int()
        lens = torch.tensor([9])
        fb = mr.prepare_forward_batch_extend(ids, torch.tensor(slots), lens, lens, torch.zeros_like(lens), loc)
        return mr.forward(fb).next_token_logits

    torch.testing.assert_close(logits(ml_dir), logits(st_dir))


def test_cpp_cpu_oracle_matches_pytorch_oracle(tmp_path):
    """The stand-alone C++ Qwen3 (no PyTorch, weights from a .mllm file) and the engine's model on the
    PyTorch statements of the ops produce the same greedy tokens and logits."""
    from mllm_b200.benchmarks.cpu_oracle import run_cpp, run_torch, seeded_weights
    from mllm_b200.models.presets import get_preset

    cfg = get_preset("qwen3-tiny", tie_word_embeddings=False)
    path = str(tmp_path / "model.mllm")
    write_mllm(path, seeded_weights(cfg, seed=1, std=0.05), model_name="tiny")
    prompt = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(1)).tolist()
    a = run_cpp(path, cfg, prompt, 6, threads=2)
    b = run_torch(path, cfg, prompt, 6)
    assert list(a["tokens"]) == b["tokens"]
    torch.testing.assert_close(torch.from_numpy(a["prefill_logits"]), b["prefill_logits"], atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(torch.from_numpy(a["last_logits"]), b["last_logits"], atol=2e-4, rtol=2e-4)


def test_quantizer_and_inspector_tools(tmp_path, capsys):
    """Block quantiser CLI -> .mllm with Q4_0 / Q8_0 entries -> the reader expands them within the
    scheme's error bound; the inspector lists dtypes, shapes and sizes."""
    from mllm_b200.io import inspect as insp
    from mllm_b200.io import quantize as quant
    from mllm_b200.io.mllm_file import MllmFileReader, write_mllm

    g = torch.Generator().manual_seed(0)
    tensors = [("model.layers.0.mlp.down_proj.weight", torch.randn(48, 64, generator=g)),
               ("model.layers.0.input_layernorm.weight", torch.ones(64)),
               ("model.embed_tokens.weight", torch.randn(100, 64, generator=g)),
               ("model.layers.0.self_attn.q_proj.weight", torch.randn(64, 96, generator=g).to(torch.bfloat16)),
               ("odd.weight", torch.randn(8, 20, generator=g))]
    src = tmp_path / "src.mllm"
    write_mllm(str(src), tensors, model_name="toy")
    for scheme, tol in (("q8_0", 1 / 127), ("q4_0", 2 / 8)):   # q4_0: half a step, a whole one where +8 clips to +7
        dst = tmp_path / f"{scheme}.mllm"
        quant.main(["--input", str(src), "--output", str(dst), "--scheme", scheme, "--model-name", "toy-q"])
        d = insp.describe(str(dst))
        kinds = {x["name"]: x["dtype"] for x in d["tensors"]}
        assert d["model_name"] == "toy-q" and d["version"] == 2
        assert kinds["model.layers.0.mlp.down_proj.weight"] == f"gguf_{scheme}"
        assert kinds["model.layers.0.self_attn.q_proj.weight"] == f"gguf_{scheme}"
        assert kinds["model.embed_tokens.weight"] == "float32" and kinds["odd.weight"] == "float32"
        assert kinds["model.layers.0.input_layernorm.weight"] == "float32"
        per_block = 34 if scheme == "q8_0" else 18
        sizes = {x["name"]: x["bytes"] for x in d["tensors"]}
        assert sizes["model.layers.0.mlp.down_proj.weight"] == 48 * 64 // 32 * per_block
        r = MllmFileReader(str(dst))
        for name, t in tensors[:1] + tensors[3:4]:
            back = r.tensor(name, torch.float32)
            assert back.shape == t.shape
            blocks = t.float().reshape(-1, 32)
            bound = blocks.abs().max(dim=1, keepdim=True).values * tol * 0.51 + 1e-3
            assert ((back.reshape(-1, 32) - blocks).abs() <= bound).all()
    insp.main([str(tmp_path / "q4_0.mllm"), "--filter", "down_proj"])
    out = capsys.readouterr().out
    assert "gguf_q4_0" in out and "down_proj" in out and "embed_tokens" not in out


def test_symmetric_heap_allocator_and_views():
    """Offset allocator of the symmetric heap (C++): deterministic first fit, alignment, coalescing;
    and the Python heap on top of it: typed views at the allocator's offsets, the same offset added to
    every rank's base."""
    import random

    from mllm_b200.parallel.symm import SymmetricHeap

    A = host_ext().SymmHeapAllocator(1 << 20, 256)
    a, b, c = A.alloc(1000), A.alloc(5000, 4096), A.alloc(100)
    assert (a, b, c) == (0, 4096, 1024) and A.used == 1024 + 5120 + 256 and A.num_blocks == 3
    assert A.free(b) and not A.free(b) and not A.free(12345)
    assert A.free(a) and A.free(c) and A.used == 0 and A.largest_free == 1 << 20     # everything merged back
    assert A.alloc(0) == -1 and A.alloc((1 << 20) + 1) == -1
    # two allocators fed the same calls agree (what makes offsets symmetric across ranks); blocks never overlap
    rng = random.Random(0)
    X, Y = host_ext().SymmHeapAllocator(1 << 16, 64), host_ext().SymmHeapAllocator(1 << 16, 64)
    live = {}
    for _ in range(2000):
        if live and rng.random() < 0.45:
            off = rng.choice(list(live))
            assert X.free(off) and Y.free(off)
            del live[off]
        else:
            n, al = rng.randrange(1, 3000), rng.choice([0, 64, 256, 1024])
            ox, oy = X.alloc(n, al), Y.alloc(n, al)
            assert ox == oy
            if ox >= 0:
                assert ox % max(al, 64) == 0 and X.block_size(ox) >= n
                for o, ln in live.items():
                    assert ox + X.block_size(ox) <= o or o + ln <= ox
                live[ox] = X.block_size(ox)
        assert X.used == sum(live.values())
    # the heap: exact capacity planning, typed views, peer addresses
    plan = [((5, 64), torch.bfloat16), ((40,), torch.int32), ((2, 3, 64), torch.bfloat16), ((7,), torch.int32)]
    heap = SymmetricHeap.local(SymmetricHeap.bytes_for(plan), world=3)
    heap.base_ptrs = [1 << 40, 2 << 40, 3 << 40]
    views = [heap.tensor(shape, dt) for shape, dt in plan]
    assert heap.alloc.used == heap.alloc.capacity
    offs = [p[0] - (1 << 40) for _, p in views]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs)
    assert heap.check_guards() == []
    for (t, ptrs), (shape, dt) in zip(views, plan):
        assert tuple(t.shape) == tuple(shape) and t.dtype == dt and t.is_contiguous()
        assert t.data_ptr() - heap.buf.data_ptr() == ptrs[0] - (1 << 40) == ptrs[2] - (3 << 40)
    views[0][0].fill_(1.5)
    views[1][0].fill_(7)
    assert float(views[0][0].sum()) == 1.5 * 320 and int(views[1][0].sum()) == 280 and int(views[3][0].sum()) == 0
    with pytest.raises(MemoryError):
        heap.tensor((1,), torch.int32)
    # canary bytes: a write one element past a buffer's end (or before its start) is reported
    assert heap.check_guards() == []
    end_of_first = offs[0] + 5 * 64 * 2
    heap.buf[end_of_first] = 0
    assert heap.check_guards() == [offs[0]]
    heap.buf[end_of_first] = 0xA5
    heap.buf[offs[2] - 1] = 7
    assert heap.check_guards() == [offs[2]]
    heap.buf[offs[2] - 1] = 0xA5
    heap.free(views[1][0])
    t, _ = heap.tensor((8,), torch.int32)
    assert t.data_ptr() == views[1][0].data_ptr()

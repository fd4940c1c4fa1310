"""tcgen05 attention kernel (prefill with cached prefixes, split decode) vs the fp32 statement."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
D = 128


def _setup(seq_lens, prefix_lens, hq, hkv, dtype=torch.bfloat16, seed=0, ctx=None):
    torch.manual_seed(seed)
    B = len(seq_lens)
    ctx = ctx or max(seq_lens) + 8
    total = sum(seq_lens)
    slots = total + 64
    kc = torch.randn(slots, hkv, D, device=DEV, dtype=dtype)
    vc = torch.randn(slots, hkv, D, device=DEV, dtype=dtype)
    rtt = torch.zeros(B + 3, ctx, dtype=torch.int32, device=DEV)
    perm = torch.randperm(slots - 1, device=DEV)[:total].int() + 1  # scattered slots: page size 1
    req = torch.arange(B, device=DEV, dtype=torch.int32) + 2
    off = 0
    for b, s in enumerate(seq_lens):
        rtt[req[b], :s] = perm[off:off + s]
        off += s
    ext = [s - p for s, p in zip(seq_lens, prefix_lens)]
    T = sum(ext)
    q = torch.randn(T, hq, D, device=DEV, dtype=dtype)
    q_start = torch.tensor([sum(ext[:i]) for i in range(B)], dtype=torch.int32, device=DEV)
    return dict(q=q, kc=kc, vc=vc, rtt=rtt, req=req, seq=torch.tensor(seq_lens, dtype=torch.int32, device=DEV),
                pre=torch.tensor(prefix_lens, dtype=torch.int32, device=DEV), q_start=q_start, max_q=max(ext))


def _err(a, b):
    return (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("seq_lens,prefix_lens", [
    ([1], [0]), ([2], [0]), ([3], [0]), ([17], [0]), ([64], [0]), ([65], [0]), ([127, 128, 129], [0, 0, 0]),
    ([300], [0]), ([700, 33], [0, 0]),
    ([200, 130], [64, 1]), ([513], [511]), ([1000], [873]),
])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (16, 8), (4, 4), (8, 1)])
def test_prefill(seq_lens, prefix_lens, hq, hkv):
    s = _setup(seq_lens, prefix_lens, hq, hkv)
    scale = D ** -0.5
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"])
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale)
    assert _err(got, want) < 3e-2


def test_prefill_strided_q_fp16():
    """q as a view into a fused qkv activation (row stride larger than Hq*D), fp16."""
    hq, hkv = 8, 2
    s = _setup([90, 200], [0, 40], hq, hkv, dtype=torch.float16, seed=3)
    T = s["q"].shape[0]
    qkv = torch.randn(T, (hq + 2 * hkv) * D, device=DEV, dtype=torch.float16)
    qkv[:, : hq * D] = s["q"].view(T, -1)
    qv = qkv[:, : hq * D].view(T, hq, D)
    got = ops.attention_prefill(qv, s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], D ** -0.5,
                                max_q_len=s["max_q"])
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], D ** -0.5)
    ops.check_status()
    assert _err(got, want) < 2e-2


@pytest.mark.parametrize("seq_lens", [[1], [2], [63], [64], [65], [500], [2048], [1, 700, 64, 129], [3000] * 3, list(range(1, 34))])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (8, 1), (4, 4)])
def test_decode(seq_lens, hq, hkv):
    s = _setup(seq_lens, [x - 1 for x in seq_lens], hq, hkv, seed=1)
    scale = D ** -0.5
    got = ops.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale, max_seq_len=max(seq_lens))
    ops.check_status()
    want = ref.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale)
    assert _err(got, want) < 3e-2


def test_decode_fixed_split_bound():
    """Graph-style call: the split count comes from the context bound, not the live lengths."""
    s = _setup([5, 900], [4, 899], 16, 8, seed=2, ctx=4096)
    got = ops.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], D ** -0.5, max_seq_len=4096)
    ops.check_status()
    want = ref.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], D ** -0.5)
    assert _err(got, want) < 3e-2


def test_large_scores_rescale():
    """Scores that grow along the sequence force the lazy rescale of the output accumulator."""
    hq = hkv = 2
    s = _setup([400], [0], hq, hkv, seed=5)
    ramp = torch.linspace(0.2, 6.0, 400, device=DEV).view(-1, 1, 1)
    s["kc"][s["rtt"][2, :400].long()] = (s["kc"][s["rtt"][2, :400].long()].float() * ramp).bfloat16()
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], 1.0,
                                max_q_len=400)
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], 1.0)
    ops.check_status()
    assert _err(got, want) < 5e-2


def _head_major(s, pattern: str, seed=0):
    """The caches of ``s`` re-stored head-major ([kv heads, slots, D] storage, handed out as [slots, kv heads, D]
    views, as the KV pool does) and the request table rewritten so that the requests' slots are runs of
    consecutive slots (``runs``), runs of 16 with scattered pages (``pages``), or a mix where every other group
    of 16 is scattered (``mixed``)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    seq = s["seq"].tolist()
    hkv = s["kc"].shape[1]
    total = sum(-(-n // 16) * 16 for n in seq) + 64
    kc = torch.randn(hkv, total, D, device=DEV, dtype=s["kc"].dtype).transpose(0, 1)
    vc = torch.randn(hkv, total, D, device=DEV, dtype=s["kc"].dtype).transpose(0, 1)
    rtt = torch.zeros_like(s["rtt"])
    pages = torch.randperm((total - 16) // 16, generator=g) + 1     # page 0 unused
    nxt = 0
    for b, n in enumerate(seq):
        np_ = -(-n // 16)
        mine = pages[nxt:nxt + np_]
        nxt += np_
        if pattern == "runs":      # one run of consecutive pages per request
            mine = torch.arange(np_) + 1 + sum(-(-m // 16) for m in seq[:b])
        slots = (mine.view(-1, 1) * 16 + torch.arange(16).view(1, -1)).reshape(-1)[:n].clone()
        if pattern == "mixed":
            for gi in range(1, np_, 2):
                lo, hi = gi * 16, min(n, gi * 16 + 16)
                slots[lo:hi] = slots[lo:hi][torch.randperm(hi - lo, generator=g)]
        rtt[s["req"][b], :n] = slots.to(DEV).int()
    return dict(s, kc=kc, vc=vc, rtt=rtt)


@pytest.mark.parametrize("pattern", ["runs", "pages", "mixed"])
@pytest.mark.parametrize("seq_lens", [[1], [15], [16], [17], [129], [500], [2048], [1, 700, 64, 129], [3000] * 3])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (8, 1)])
def test_decode_head_major_pool(pattern, seq_lens, hq, hkv):
    """Decode over head-major storage: groups of 16 consecutive slots arrive as whole boxes, scattered groups row
    by row; both must give the fp32 statement's result."""
    s = _head_major(_setup(seq_lens, [x - 1 for x in seq_lens], hq, hkv, seed=1), pattern, seed=len(seq_lens))
    assert s["kc"].stride(0) == D and (hkv == 1 or not s["kc"].is_contiguous())
    scale = D ** -0.5
    got = ops.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale, max_seq_len=max(seq_lens))
    ops.check_status()
    want = ref.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("seq_lens,prefix_lens", [([300], [0]), ([200, 130], [64, 1]), ([1000], [873])])
def test_prefill_head_major_pool(seq_lens, prefix_lens):
    s = _head_major(_setup(seq_lens, prefix_lens, 16, 8), "pages", seed=2)
    scale = D ** -0.5
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"])
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("pattern", ["pages", "scattered"])
def test_prefill_long_sequences_many_tiles(pattern):
    """Benchmark-like shape: enough 128-token tiles that every ring slot and barrier phase of the warp-specialised
    kernel wraps several times, with slots in pages of 16 (boxes) and scattered (row gathers)."""
    s = _setup([2048, 1500], [0, 300], 32, 8, seed=5)
    if pattern == "pages":
        s = _head_major(s, "pages", seed=4)
    scale = D ** -0.5
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"])
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("seq_lens,prefix_lens", [([3], [0]), ([700, 33], [0, 0]), ([200, 130], [64, 1])])
def test_prefill_single_role_kernel(monkeypatch, seq_lens, prefix_lens):
    """The older kernel (every warp gathers, computes the softmax and issues in turn) still serves storage that
    is neither head-major nor slot-major; the switch selects it for any storage."""
    monkeypatch.setenv("MLLM_B200_ATTN_PREFILL", "legacy")
    s = _setup(seq_lens, prefix_lens, 8, 2, seed=7)
    scale = D ** -0.5
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"])
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale)
    assert _err(got, want) < 3e-2


def test_kv_write_kernels_on_head_major_pool():
    """The stand-alone KV write and the fused norm + rotary + write kernel address the caches by strides."""
    from mllm_b200.mem_cache import KVPool

    pool = KVPool(256, 1, 4, D, torch.bfloat16, DEV)
    kc, vc = pool.get_kv_buffer(0)
    assert kc.stride(0) == D and kc.stride(1) == pool.num_slots * D
    torch.manual_seed(0)
    k = torch.randn(37, 4, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(37, 4, D, device=DEV, dtype=torch.bfloat16)
    loc = torch.randperm(255, device=DEV)[:37] + 1
    ops.kv_write(k, v, loc, kc, vc)
    ops.check_status()
    assert torch.equal(kc[loc], k) and torch.equal(vc[loc], v)
    assert torch.equal(pool.store[0, 0, 2, loc], k[:, 2])


@pytest.mark.parametrize("window,cap", [(64, 0.0), (100, 0.0), (1, 0.0), (4096, 0.0), (0, 30.0), (150, 20.0)])
@pytest.mark.parametrize("seq_lens,prefix_lens", [([300], [0]), ([700, 33], [0, 0]), ([200, 130], [64, 1]), ([1000], [873])])
def test_prefill_sliding_window_and_soft_cap(window, cap, seq_lens, prefix_lens):
    """Sliding window (each query sees its last ``window`` keys) and soft-capped scores as options of the
    tcgen05 prefill kernel, against the fp32 statement."""
    s = _setup(seq_lens, prefix_lens, 16, 8, seed=window + int(cap))
    scale = D ** -0.5 * (3.0 if cap else 1.0)      # larger scores so that the cap bites
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"], window=window or None, logit_cap=cap)
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                 window=window or None, logit_cap=cap)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("window,cap", [(64, 0.0), (129, 0.0), (1, 0.0), (5000, 0.0), (0, 30.0), (700, 20.0)])
@pytest.mark.parametrize("seq_lens", [[1], [65], [500], [2048], [1, 700, 64, 129]])
def test_decode_sliding_window_and_soft_cap(window, cap, seq_lens):
    s = _head_major(_setup(seq_lens, [x - 1 for x in seq_lens], 32, 8, seed=1), "pages", seed=3)
    scale = D ** -0.5 * (3.0 if cap else 1.0)
    got = ops.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale, max_seq_len=max(seq_lens),
                               window=window or None, logit_cap=cap)
    ops.check_status()
    want = ref.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale, window=window or None,
                                logit_cap=cap)
    assert _err(got, want) < 3e-2

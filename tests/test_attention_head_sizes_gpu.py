"""Head sizes 64 and 256 on the tcgen05 attention kernel (the single-role kernel instantiated for one and four
64-feature halves per row): prefill with cached prefixes, decode with split KV ranges, sliding window and soft cap,
slot-major and head-major pools, and the bidirectional variable-length form the vision towers use (64-wide heads,
unpadded) -- each against the fp32 statement of the same op."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(D, seq_lens, prefix_lens, hq, hkv, dtype=torch.bfloat16, seed=0, head_major=False):
    torch.manual_seed(seed)
    B = len(seq_lens)
    ctx = max(seq_lens) + 8
    total = sum(seq_lens)
    slots = total + 64
    if head_major:      # [kv heads, slots, D] storage handed out as [slots, kv heads, D] views, as the KV pool does
        kc = torch.randn(hkv, slots, D, device=DEV, dtype=dtype).transpose(0, 1)
        vc = torch.randn(hkv, slots, D, device=DEV, dtype=dtype).transpose(0, 1)
    else:
        kc = torch.randn(slots, hkv, D, device=DEV, dtype=dtype)
        vc = torch.randn(slots, hkv, D, device=DEV, dtype=dtype)
    rtt = torch.zeros(B + 3, ctx, dtype=torch.int32, device=DEV)
    perm = torch.randperm(slots - 1, device=DEV)[:total].int() + 1
    req = torch.arange(B, device=DEV, dtype=torch.int32) + 2
    off = 0
    for b, s in enumerate(seq_lens):
        rtt[req[b], :s] = perm[off:off + s]
        off += s
    ext = [s - p for s, p in zip(seq_lens, prefix_lens)]
    q = torch.randn(sum(ext), hq, D, device=DEV, dtype=dtype)
    q_start = torch.tensor([sum(ext[:i]) for i in range(B)], dtype=torch.int32, device=DEV)
    return dict(q=q, kc=kc, vc=vc, rtt=rtt, req=req, seq=torch.tensor(seq_lens, dtype=torch.int32, device=DEV),
                pre=torch.tensor(prefix_lens, dtype=torch.int32, device=DEV), q_start=q_start, max_q=max(ext))


def _err(a, b):
    return (a.float() - b.float()).abs().max().item()


def _ran_on_kernels(before):
    assert ops.launch_count() > before, "the attention call did not launch one of the package's kernels"


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("seq_lens,prefix_lens", [
    ([1], [0]), ([3], [0]), ([64], [0]), ([65], [0]), ([127, 128, 129], [0, 0, 0]), ([700, 33], [0, 0]),
    ([200, 130], [64, 1]), ([1000], [873]),
])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (4, 4), (8, 1)])
def test_prefill(D, seq_lens, prefix_lens, hq, hkv):
    s = _setup(D, seq_lens, prefix_lens, hq, hkv)
    scale = D ** -0.5
    n0 = ops.launch_count()
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"])
    ops.check_status()
    _ran_on_kernels(n0)
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("D", [64, 256])
def test_prefill_head_major_pool_fp16_strided_q(D):
    hq, hkv = 8, 2
    s = _setup(D, [90, 300], [0, 40], hq, hkv, dtype=torch.float16, seed=3, head_major=True)
    T = s["q"].shape[0]
    qkv = torch.randn(T, (hq + 2 * hkv) * D, device=DEV, dtype=torch.float16)
    qkv[:, : hq * D] = s["q"].view(T, -1)
    qv = qkv[:, : hq * D].view(T, hq, D)
    got = ops.attention_prefill(qv, s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], D ** -0.5,
                                max_q_len=s["max_q"])
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], D ** -0.5)
    assert _err(got, want) < 2e-2


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("seq_lens", [[1], [63], [64], [65], [500], [2048], [1, 700, 64, 129], [3000] * 3])
@pytest.mark.parametrize("hq,hkv,head_major", [(32, 8, True), (8, 1, False), (4, 4, True)])
def test_decode(D, seq_lens, hq, hkv, head_major):
    s = _setup(D, seq_lens, [x - 1 for x in seq_lens], hq, hkv, seed=1, head_major=head_major)
    scale = D ** -0.5
    n0 = ops.launch_count()
    got = ops.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale, max_seq_len=max(seq_lens))
    ops.check_status()
    _ran_on_kernels(n0)
    want = ref.attention_decode(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], scale)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("window,cap", [(64, 0.0), (100, 0.0), (0, 30.0), (150, 20.0)])
def test_sliding_window_and_soft_cap(D, window, cap):
    s = _setup(D, [700, 33, 300], [0, 0, 100], 8, 4, seed=window + int(cap))
    scale = D ** -0.5 * (3.0 if cap else 1.0)
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                max_q_len=s["max_q"], window=window or None, logit_cap=cap)
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], scale,
                                 window=window or None, logit_cap=cap)
    assert _err(got, want) < 3e-2
    d = _setup(D, [500, 65, 2048], [499, 64, 2047], 8, 4, seed=5)
    got = ops.attention_decode(d["q"], d["kc"], d["vc"], d["rtt"], d["req"], d["seq"], scale, max_seq_len=2048,
                               window=window or None, logit_cap=cap)
    ops.check_status()
    want = ref.attention_decode(d["q"], d["kc"], d["vc"], d["rtt"], d["req"], d["seq"], scale, window=window or None,
                                logit_cap=cap)
    assert _err(got, want) < 3e-2


@pytest.mark.parametrize("D", [64, 256])
def test_large_scores_rescale(D):
    """Scores that grow along the sequence force the lazy rescale of the accumulator in tensor memory."""
    s = _setup(D, [600], [0], 4, 2, seed=7)
    ramp = torch.linspace(0.2, 3.0, s["kc"].shape[0], device=DEV).view(-1, 1, 1)
    s["kc"] = (s["kc"].float() * ramp).to(s["kc"].dtype)
    got = ops.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], 0.5,
                                max_q_len=s["max_q"])
    ops.check_status()
    want = ref.attention_prefill(s["q"], s["kc"], s["vc"], s["rtt"], s["req"], s["seq"], s["pre"], s["q_start"], 0.5)
    assert _err(got, want) < 5e-2


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("lens", [[196], [64, 1, 300], [1024, 77]])
def test_bidirectional_varlen(D, lens):
    torch.manual_seed(2)
    T, H = sum(lens), 4
    q, k, v = (torch.randn(T, H, D, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    n0 = ops.launch_count()
    got = ops.attention_varlen_bidirectional(q, k, v, cu, D ** -0.5)
    ops.check_status()
    _ran_on_kernels(n0)
    want = ref.attention_varlen_bidirectional(q.float(), k.float(), v.float(), cu, D ** -0.5)
    assert got.shape == (T, H, D) and _err(got, want) < 3e-2


def test_vision_attention_runs_64_wide_heads_unpadded():
    torch.manual_seed(3)
    T, H, D = 320, 4, 64
    qkv = torch.randn(T, 3 * H * D, device=DEV, dtype=torch.bfloat16)
    ang = torch.rand(T, D // 2, device=DEV) * 6.0
    cos, sin = ang.cos(), ang.sin()
    cu = torch.tensor([0, 196, 320], dtype=torch.int32)
    got = ops.vision_attention(qkv, cos, sin, cu, H, D ** -0.5)
    ops.check_status()
    q, k, v = qkv.float().view(T, 3, H, D).unbind(1)
    q, k = ref.vision_rope(q, cos, sin), ref.vision_rope(k, cos, sin)
    want = ref.attention_varlen_bidirectional(q, k, v, cu, D ** -0.5).reshape(T, H * D)
    assert _err(got, want) < 3e-2

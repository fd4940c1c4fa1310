"""sm_100a element-wise kernels against the fp32 PyTorch statement of the same op."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol=2e-2, rtol=2e-2):
    torch.testing.assert_close(a.float(), b.float(), atol=atol, rtol=rtol)


@pytest.mark.parametrize("rows,hidden", [(1, 1024), (3, 4096), (17, 5120), (129, 2048), (2, 8192)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rmsnorm(rows, hidden, dtype):
    torch.manual_seed(0)
    x = torch.randn(rows, hidden, device=DEV, dtype=dtype)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype)
    _close(ops.rmsnorm(x, w, 1e-6), ref.rmsnorm(x, w, 1e-6))


@pytest.mark.parametrize("rows,hidden", [(1, 1024), (7, 4096), (128, 5120)])
def test_fused_add_rmsnorm(rows, hidden):
    torch.manual_seed(1)
    x = torch.randn(rows, hidden, device=DEV, dtype=torch.bfloat16)
    r = torch.randn(rows, hidden, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).bfloat16()
    x2, r2 = x.clone(), r.clone()
    ops.fused_add_rmsnorm(x, r, w, 1e-6)
    ref.fused_add_rmsnorm(x2, r2, w, 1e-6)
    assert torch.equal(r, r2)  # the sum is rounded once, identically
    _close(x, x2)


def test_layernorm():
    torch.manual_seed(2)
    x = torch.randn(33, 1024, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(1024, device=DEV).bfloat16()
    b = torch.randn(1024, device=DEV).bfloat16()
    _close(ops.layernorm(x, w, b, 1e-6), ref.layernorm(x, w, b, 1e-6), atol=3e-2)


@pytest.mark.parametrize("rows,inter", [(1, 3072), (5, 12288), (200, 768)])
def test_act_and_mul(rows, inter):
    torch.manual_seed(3)
    x = torch.randn(rows, 2 * inter, device=DEV, dtype=torch.bfloat16)
    _close(ops.silu_and_mul(x), ref.silu_and_mul(x))
    _close(ops.gelu_tanh_and_mul(x), ref.gelu_tanh_and_mul(x))
    _close(ops.gelu_tanh(x), ref.gelu_tanh(x))


def test_embedding():
    torch.manual_seed(4)
    table = torch.randn(1000, 2048, device=DEV, dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (37,), device=DEV)
    assert torch.equal(ops.embedding(ids, table), table[ids])


# long batches: a warp then owns several heads of its token (every 10th, every 2nd, all of them)
@pytest.mark.parametrize("tokens", [1, 2, 3, 17, 127, 128, 129, 3000, 16384, 40000])
@pytest.mark.parametrize("hq,hkv", [(16, 8), (32, 8), (4, 1)])
def test_qk_norm_rope_kv_write(tokens, hq, hkv):
    torch.manual_seed(5)
    D = 128
    qkv = torch.randn(tokens, (hq + 2 * hkv) * D, device=DEV, dtype=torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    pos = torch.randint(0, 4096, (tokens,), device=DEV)
    slots = max(300, tokens + 8)
    loc = torch.randperm(slots - 1, device=DEV)[:tokens] + 1
    kc = torch.zeros(slots, hkv, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qkv2, kc2, vc2 = qkv.clone(), kc.clone(), vc.clone()
    ops.qk_norm_rope_kv_write(qkv, qw, kw, pos, loc, kc, vc, hq, hkv, D, 1e6, 1e-6)
    ref.qk_norm_rope_kv_write(qkv2, qw, kw, pos, loc, kc2, vc2, hq, hkv, D, 1e6, 1e-6)
    _close(qkv, qkv2, atol=3e-2, rtol=3e-2)
    _close(kc, kc2, atol=3e-2, rtol=3e-2)
    assert torch.equal(vc, vc2)
    ops.check_status()


def test_mrope_variant():
    torch.manual_seed(6)
    D, hq, hkv, T = 128, 8, 2, 50
    qkv = torch.randn(T, (hq + 2 * hkv) * D, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (3, T), device=DEV)
    loc = torch.arange(1, T + 1, device=DEV)
    kc = torch.zeros(64, hkv, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for inter in (True, False):
        a, b = qkv.clone(), qkv.clone()
        kc1, vc1, kc2, vc2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
        ops.qk_norm_rope_kv_write(a, None, None, pos, loc, kc1, vc1, hq, hkv, D, 5e6, 1e-6, [24, 20, 20], inter)
        ref.qk_norm_rope_kv_write(b, None, None, pos, loc, kc2, vc2, hq, hkv, D, 5e6, 1e-6, [24, 20, 20], inter)
        _close(a, b, atol=3e-2, rtol=3e-2)
        _close(kc1, kc2, atol=3e-2, rtol=3e-2)


def test_kv_write_exact():
    torch.manual_seed(7)
    k = torch.randn(19, 8, 128, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(19, 8, 128, device=DEV, dtype=torch.bfloat16)
    loc = torch.randperm(99, device=DEV)[:19] + 1
    kc = torch.zeros(100, 8, 128, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    ops.kv_write(k, v, loc, kc, vc)
    assert torch.equal(kc[loc], k) and torch.equal(vc[loc], v)


def test_per_token_quant_int8():
    torch.manual_seed(8)
    x = torch.randn(45, 4096, device=DEV, dtype=torch.bfloat16) * 3
    q, s = ops.per_token_quant_int8(x)
    q2, s2 = ref.per_token_quant_int8(x)
    torch.testing.assert_close(s, s2, rtol=1e-6, atol=0)
    assert (q.int() - q2.int()).abs().max() <= 1
    assert (q != q2).float().mean() < 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_argmax(dtype):
    torch.manual_seed(9)
    logits = torch.randn(9, 151936, device=DEV, dtype=dtype)
    logits[3, 77] = 100.0
    logits[4, 151935] = 100.0
    got = ops.argmax(logits)
    want = torch.argmax(logits.float(), dim=-1)
    # bf16 ties: the kernel returns the lowest index among equal maxima
    assert torch.equal(logits.float().gather(1, got[:, None]), logits.float().gather(1, want[:, None]))
    assert got[3] == 77 and got[4] == 151935

"""tcgen05 GEMM (bf16 / fp16 / int8, normal and small-batch tilings) against fp32 references."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(got, want):
    return ((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-6)).item()


SHAPES = [
    # (m, n, k)
    (1, 1024, 1024), (2, 4096, 4096), (3, 6144, 4096), (17, 4096, 12288), (32, 1024, 3072),
    (127, 2048, 1024), (128, 4096, 1024), (129, 1024, 2048), (256, 4096, 4096),
    (257, 1024, 1024), (512, 4096, 4096), (1000, 2048, 1024), (2048, 6144, 4096), (4096, 4096, 12288),
    (300, 1000, 520),  # ragged n (multiple of 8) and k (multiple of 8)
    (5, 151936, 1024),  # lm_head
]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_bf16(m, n, k):
    torch.manual_seed(m * 7 + n + k)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * (k ** -0.5)
    got = ops.linear(x, w)
    ops.check_status()
    want = ref.linear(x, w, out_dtype=torch.float32)
    assert _rel_err(got, want) < 6e-3


@pytest.mark.parametrize("m", [4, 64, 300, 1024])
def test_gemm_fp16_bias_residual(m):
    torch.manual_seed(m)
    n, k = 2048, 1024
    x = torch.randn(m, k, device=DEV, dtype=torch.float16)
    w = torch.randn(n, k, device=DEV, dtype=torch.float16) * (k ** -0.5)
    b = torch.randn(n, device=DEV, dtype=torch.float16)
    r = torch.randn(m, n, device=DEV, dtype=torch.float16)
    got = ops.linear(x, w, bias=b, residual=r)
    ops.check_status()
    want = ref.linear(x, w, b, r, out_dtype=torch.float32)
    assert _rel_err(got, want) < 2e-3


@pytest.mark.parametrize("m", [1, 8, 33, 256, 300, 2048])
@pytest.mark.parametrize("inter,k", [(3072, 1024), (768, 2048)])
def test_gemm_swiglu(m, inter, k):
    torch.manual_seed(m + inter)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(2 * inter, k, device=DEV, dtype=torch.bfloat16) * (k ** -0.5)  # [gate ; up]
    wi = ref.interleave_gate_up(w, ops.SWIGLU_BLOCK).contiguous()
    got = ops.linear_swiglu(x, wi)
    ops.check_status()
    want = ref.linear_swiglu(x.float(), w.float(), 0)
    assert _rel_err(got, want) < 8e-3
    # the interleave helper itself
    torch.testing.assert_close(ref.linear_swiglu(x, wi, ops.SWIGLU_BLOCK).float(), want.bfloat16().float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("m,n,k", [(1, 1024, 1024), (16, 4096, 4096), (200, 2048, 3072), (512, 6144, 2048), (2048, 4096, 4096)])
def test_gemm_w8a8(m, n, k):
    torch.manual_seed(m + n)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    wq = torch.randint(-127, 128, (n, k), device=DEV, dtype=torch.int8)
    ws = torch.rand(n, device=DEV) * 0.01 + 0.001
    xq, xs = ops.per_token_quant_int8(x)
    got = ops.int8_scaled_mm(xq, wq, xs, ws, torch.bfloat16)
    ops.check_status()
    acc = torch._int_mm(xq, wq.t()) if m > 16 and m % 8 == 0 else (xq.float() @ wq.float().t())
    want = acc.float() * xs.reshape(-1, 1) * ws.reshape(1, -1)
    assert _rel_err(got, want) < 6e-3


def test_gemm_repeatable_splitk():
    """Split-K tickets reset themselves: the same small-batch GEMM gives identical bits twice."""
    torch.manual_seed(0)
    x = torch.randn(4, 12288, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(4096, 12288, device=DEV, dtype=torch.bfloat16) * 0.01
    a = ops.linear(x, w)
    b = ops.linear(x, w)
    ops.check_status()
    assert torch.equal(a, b)


@pytest.mark.parametrize("m,n,k,dtype", [(2500, 4096, 1024, torch.float16), (4096, 2048, 4096, torch.bfloat16),
                                         (16384, 1024, 512, torch.bfloat16)])
def test_gemm_two_cta_tiles_bias_residual_ragged_rows(m, n, k, dtype):
    """Shapes with enough 256 x 256 tiles for the two-CTA tiling; m = 2500 leaves a partial last row tile."""
    torch.manual_seed(m + n)
    x = torch.randn(m, k, device=DEV, dtype=dtype)
    w = torch.randn(n, k, device=DEV, dtype=dtype) * (k ** -0.5)
    b = torch.randn(n, device=DEV, dtype=dtype)
    r = torch.randn(m, n, device=DEV, dtype=dtype)
    got = ops.linear(x, w, bias=b, residual=r)
    ops.check_status()
    want = ref.linear(x, w, b, r, out_dtype=torch.float32)
    assert _rel_err(got, want) < (2e-3 if dtype == torch.float16 else 6e-3)
    got2 = ops.linear(x, w)
    ops.check_status()
    assert _rel_err(got2, ref.linear(x, w, out_dtype=torch.float32)) < 6e-3


@pytest.mark.parametrize("m,n,k", [(1, 1024, 1024), (8, 6144, 4096), (8, 4096, 12288), (40, 2048, 1024), (200, 4096, 4096)])
def test_gemm_small_batch_with_parameter_weights(m, n, k):
    """Weights held in an ``nn.Parameter`` take the path that starts the weight stream ahead of the
    stream-order wait; several launches back to back (each waits on the one before) must all be right."""
    torch.manual_seed(m + n + k)
    w = torch.nn.Parameter(torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * (k ** -0.5), requires_grad=False)
    xs = [torch.randn(m, k, device=DEV, dtype=torch.bfloat16) for _ in range(4)]
    outs = [ops.linear(x, w) for x in xs]
    ops.check_status()
    for x, got in zip(xs, outs):
        assert _rel_err(got, ref.linear(x, w.data, out_dtype=torch.float32)) < 6e-3
    # a chain: each GEMM consumes the previous one's output, so an early start must still see it
    w2 = torch.nn.Parameter(torch.randn(k, n, device=DEV, dtype=torch.bfloat16) * (n ** -0.5), requires_grad=False)
    y = xs[0]
    want = xs[0].float()
    for _ in range(3):
        y = ops.linear(ops.linear(y, w), w2)
        want = ref.linear(ref.linear(want.bfloat16(), w.data, out_dtype=torch.float32).bfloat16(), w2.data,
                          out_dtype=torch.float32)
    ops.check_status()
    assert _rel_err(y, want) < 3e-2


@pytest.mark.parametrize("m", [1, 2, 5, 8])
@pytest.mark.parametrize("n,k", [(4096, 4096), (6144, 4096), (4096, 12288), (1024, 6144), (6144, 8192), (1024, 256), (8, 512),
                                 (151936, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_streaming_gemm_for_a_handful_of_rows(m, n, k, dtype):
    """Up to 8 rows and k a multiple of 256 take the register-streaming kernel (weights through warp-level MMAs,
    no tensor memory); with a Parameter its weight loads go out before the stream-order wait."""
    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device=DEV, dtype=dtype)
    w = torch.nn.Parameter(torch.randn(n, k, device=DEV, dtype=dtype) * (k ** -0.5), requires_grad=False)
    b = torch.randn(n, device=DEV, dtype=dtype)
    r = torch.randn(m, n, device=DEV, dtype=dtype)
    want = ref.linear(x, w.data, out_dtype=torch.float32)
    assert _rel_err(ops.linear(x, w), want) < 6e-3
    assert _rel_err(ops.linear(x, w, bias=b, residual=r), ref.linear(x, w.data, b, r, out_dtype=torch.float32)) < 6e-3
    # activations as a view with a larger row stride, plain-tensor weights
    wide = torch.randn(m, k + 64, device=DEV, dtype=dtype)
    assert _rel_err(ops.linear(wide[:, :k], w.data), ref.linear(wide[:, :k], w.data, out_dtype=torch.float32)) < 6e-3
    ops.check_status()


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("inter,k", [(12288, 4096), (768, 2048), (128, 256)])
def test_streaming_gemm_swiglu(m, inter, k):
    torch.manual_seed(m + inter)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(2 * inter, k, device=DEV, dtype=torch.bfloat16) * (k ** -0.5)  # [gate ; up]
    wi = torch.nn.Parameter(ref.interleave_gate_up(w, ops.SWIGLU_BLOCK).contiguous(), requires_grad=False)
    got = ops.linear_swiglu(x, wi)
    ops.check_status()
    want = ref.linear_swiglu(x.float(), w.float(), 0)
    assert _rel_err(got, want) < 8e-3


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("n,k,swiglu", [(6144, 4096, False), (24576, 4096, True), (1024, 1024, False), (512, 2048, True)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_add_rmsnorm_fused_into_the_streaming_gemm(monkeypatch, m, n, k, swiglu, with_residual):
    """residual add + RMSNorm as the prologue of the small-batch GEMM: one launch gives the product of the normed
    rows and the new residual stream; checked against the fp32 statement of the three steps."""
    monkeypatch.setattr(ops, "_FUSE_NORM_GEMM", True)
    torch.manual_seed(m + n + k)
    dt = torch.bfloat16
    x = torch.randn(m, k, device=DEV, dtype=dt)
    res = torch.randn(m, k, device=DEV, dtype=dt) if with_residual else None
    nw = (1 + 0.1 * torch.randn(k, device=DEV)).to(dt)
    w = torch.randn(n, k, device=DEV, dtype=dt) * (k ** -0.5)
    wk = torch.nn.Parameter(ref.interleave_gate_up(w, ops.SWIGLU_BLOCK).contiguous() if swiglu else w, requires_grad=False)
    res_before = None if res is None else res.clone()
    y, s = ops.add_rmsnorm_linear(x, res, nw, 1e-6, wk, swiglu=swiglu)
    ops.check_status()
    if res is not None:
        assert torch.equal(res, res_before), "the fused path must not touch the incoming residual"
    s_want = (x.float() + (res.float() if res is not None else 0)).to(dt)
    assert torch.equal(s, s_want)
    h = (s_want.float() * torch.rsqrt(s_want.float().pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(dt)
    want = ref.linear_swiglu(h.float(), w.float(), 0) if swiglu else ref.linear(h, w, out_dtype=torch.float32)
    assert _rel_err(y, want) < 8e-3
    # an input the fused kernel does not take (9 rows) goes through the separate kernels with the same result
    x9 = torch.randn(9, k, device=DEV, dtype=dt)
    r9 = torch.randn(9, k, device=DEV, dtype=dt)
    s9_want = (x9.float() + r9.float()).to(dt)
    y9, s9 = ops.add_rmsnorm_linear(x9.clone(), r9, nw, 1e-6, wk, swiglu=swiglu)
    assert torch.equal(s9, s9_want)
    h9 = (s9_want.float() * torch.rsqrt(s9_want.float().pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(dt)
    want9 = ref.linear_swiglu(h9.float(), w.float(), 0) if swiglu else ref.linear(h9, w, out_dtype=torch.float32)
    assert _rel_err(y9, want9) < 8e-3

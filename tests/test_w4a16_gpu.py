"""W4A16 tcgen05 GEMM (in-kernel nibble expansion) against the fp32 dequantise-then-matmul statement."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _case(M, N, K, group, zeros, bias, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    qw = torch.randint(-(2 ** 31), 2 ** 31 - 1, (N, K // 8), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    sc = (torch.rand(N, K // group, device="cuda", generator=g) * 0.02 + 0.005).to(dtype)
    z = torch.randint(0, 16, (N, K // group), device="cuda", generator=g, dtype=torch.int64).to(torch.uint8) if zeros else None
    b = torch.randn(N, device="cuda", generator=g).to(dtype) if bias else None
    return x, qw, sc, z, b


@pytest.mark.parametrize("M", [1, 8, 40, 130, 300, 1000])
@pytest.mark.parametrize("N,K,group", [(256, 512, 128), (384, 2048, 128), (2048, 1024, 64), (200, 256, 128)])
def test_w4a16_matches_reference(M, N, K, group):
    x, qw, sc, z, b = _case(M, N, K, group, zeros=False, bias=False, dtype=torch.bfloat16, seed=M + N)
    got = ops.w4a16_gemm(x, qw, sc, None, group).float()
    w = ref.dequant_w4(qw, sc, None, group).to(torch.bfloat16).float()   # the kernel rounds expanded weights once
    want = x.float() @ w.t()
    ops.check_status()
    assert (got - want).abs().max().item() <= 0.02 * want.abs().max().item() + 0.02


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [4, 500])
def test_w4a16_zero_points_and_bias(dtype, M):
    N, K, group = 512, 1024, 128
    x, qw, sc, z, b = _case(M, N, K, group, zeros=True, bias=True, dtype=dtype, seed=7)
    got = ops.w4a16_gemm(x, qw, sc, z, group, b).float()
    w = ref.dequant_w4(qw, sc, z, group).to(dtype).float()
    want = x.float() @ w.t() + b.float()
    ops.check_status()
    assert (got - want).abs().max().item() <= 0.02 * want.abs().max().item() + 0.02


def test_w4a16_expansion_is_exact():
    """With a one-hot activation row the output is a column of the expanded weight matrix: it must equal
    round_to_bf16((q - 8) * scale) exactly."""
    N, K, group = 256, 256, 128
    x = torch.zeros(16, K, device="cuda", dtype=torch.bfloat16)
    cols = torch.arange(16, device="cuda") * 13 % K
    x[torch.arange(16), cols] = 1.0
    _, qw, sc, _, _ = _case(1, N, K, group, False, False, torch.bfloat16, seed=3)
    got = ops.w4a16_gemm(x, qw, sc, None, group)
    w = ref.dequant_w4(qw, sc.float(), None, group)
    want = w.to(torch.bfloat16)[:, cols].t()
    assert torch.equal(got, want)


@pytest.mark.parametrize("M,N,K,group,zeros,dtype", [(8, 512, 1024, 128, False, torch.bfloat16), (8, 4096, 4096, 128, True, torch.bfloat16),
                                                     (300, 384, 2048, 64, True, torch.float16), (1, 256, 256, 128, False, torch.bfloat16)])
def test_w4a16_interleaved_nibbles_give_the_same_bits(M, N, K, group, zeros, dtype):
    """The loaders re-order the nibbles of every word for the kernel's fast expansion; the product must be
    bit-identical to the natural-order path on the same weights."""
    x, qw, sc, z, b = _case(M, N, K, group, zeros=zeros, bias=True, dtype=dtype, seed=M + K)
    natural = ops.w4a16_gemm(x, qw, sc, z, group, b)
    il = ops.w4a16_interleave(qw)
    assert torch.equal(ops.w4a16_deinterleave(il), qw)
    fast = ops.w4a16_gemm(x, il, sc, z, group, b, interleaved=True)
    ops.check_status()
    assert torch.equal(natural, fast)


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("N,K,group", [(4096, 4096, 128), (6144, 4096, 128), (1024, 1024, 32), (512, 2048, 64), (24576, 4096, 128),
                                       (4096, 12288, 128), (1024, 6144, 64), (256, 8192, 128)])
@pytest.mark.parametrize("zeros,interleaved,dtype", [(False, True, torch.bfloat16), (True, False, torch.bfloat16),
                                                     (True, True, torch.float16)])
def test_w4a16_streaming_kernel_for_a_handful_of_rows(M, N, K, group, zeros, interleaved, dtype):
    """Up to 8 rows; k a multiple of 1024 up to 4096 (two CTAs per SM), or a multiple of 2048 up to 12288 (one CTA
    whose shared memory is mostly the activation rows): weights, scales and zero points stream through a per-lane
    copy queue and are expanded in registers (no tensor memory); against the fp32 statement."""
    x, qw, sc, z, b = _case(M, N, K, group, zeros=zeros, bias=True, dtype=dtype, seed=M + N + K)
    w = ref.dequant_w4(qw, sc, z, group).to(dtype).float()
    want = x.float() @ w.t() + b.float()
    q_in = ops.w4a16_interleave(qw) if interleaved else qw
    got = ops.w4a16_gemm(x, q_in, sc, z, group, b, interleaved=interleaved).float()
    ops.check_status()
    assert (got - want).abs().max().item() <= 0.02 * want.abs().max().item() + 0.02

"""Sampling semantics (CPU) and the sort-free sampling kernel against them (GPU)."""
import pytest
import torch

from mllm_b200 import ops
from mllm_b200.ops import reference as ref


def _params(B, temp=1.0, k=0, p=1.0, device="cpu"):
    return (torch.full((B,), temp, device=device), torch.full((B,), k, dtype=torch.int32, device=device),
            torch.full((B,), p, device=device))


def test_reference_filters():
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.125, 0.0625, 0.0625]]))
    t, k, p = _params(1)
    # no filter: inverse CDF in id order
    for u, want in [(0.0, 0), (0.49, 0), (0.51, 1), (0.76, 2), (0.99, 4)]:
        assert int(ref.top_k_top_p_min_p_sample(logits, t, k, p, None, torch.tensor([u]))) == want
    # top-k 2 keeps ids {0, 1} with masses 2/3, 1/3
    t, k, p = _params(1, k=2)
    assert int(ref.top_k_top_p_min_p_sample(logits, t, k, p, None, torch.tensor([0.7]))) == 1
    assert int(ref.top_k_top_p_min_p_sample(logits, t, k, p, None, torch.tensor([0.999]))) == 1
    # top-p 0.7: mass before id 2 is 0.75 >= 0.7 -> ids {0, 1}
    t, k, p = _params(1, p=0.7)
    assert int(ref.top_k_top_p_min_p_sample(logits, t, k, p, None, torch.tensor([0.999]))) == 1
    # min-p 0.3 (relative to the max): 0.125/0.5 = 0.25 < 0.3 -> ids {0, 1}
    t, k, p = _params(1)
    assert int(ref.top_k_top_p_min_p_sample(logits, t, k, p, torch.tensor([0.3]), torch.tensor([0.999]))) == 1
    # ties at the cut-off are all kept: top-k 4 keeps both 0.0625 entries
    t, k, p = _params(1, k=4)
    assert int(ref.top_k_top_p_min_p_sample(logits, t, k, p, None, torch.tensor([0.999]))) == 4
    # greedy
    t, k, p = _params(1, temp=0.0)
    assert int(ref.top_k_top_p_min_p_sample(logits, t, k, p, None, torch.tensor([0.9]))) == 0


def test_reference_penalties():
    logits = torch.tensor([[2.0, -1.0, 0.5, 1.0]])
    counts = torch.tensor([[2, 0, 1, 0]])
    pm = torch.tensor([[False, True, False, False]])
    out = ref.apply_penalties(logits, counts, pm, torch.tensor([0.5]), torch.tensor([0.25]), torch.tensor([2.0]))
    want = torch.tensor([[(2.0 - 1.0 - 0.25) / 2, -1.0 * 2, (0.5 - 0.5 - 0.25) * 2, 1.0]])
    torch.testing.assert_close(out, want)


def _check_row(logits_row, temp, k, p, mp, u, tok):
    """The kernel's token must lie in the reference kept set and bracket the target mass, with slack for
    fp32-vs-fp64 rounding at the cut-off and in the running sum."""
    row = logits_row.double().cpu()
    e = torch.exp((row - row.max()) / temp)
    se = torch.sort(e, descending=True).values
    tau = 0.0
    V = row.numel()
    if 0 < k < V:
        tau = max(tau, float(se[k - 1]))
    if p < 1.0:
        before = torch.cumsum(se, 0) - se
        n = int((before < p * float(se.sum())).sum())
        tau = max(tau, float(se[max(n, 1) - 1]))
    if mp > 0:
        tau = max(tau, mp)
    assert float(e[tok]) >= tau * (1 - 1e-4), (float(e[tok]), tau)
    strict = torch.where(e >= tau * (1 + 1e-4), e, torch.zeros_like(e))
    loose = torch.where(e >= tau * (1 - 1e-4), e, torch.zeros_like(e))
    lo = float(torch.cumsum(strict, 0)[tok - 1]) if tok > 0 else 0.0
    hi = float(torch.cumsum(loose, 0)[tok])
    slack = 2e-3 * float(loose.sum())
    assert u * float(loose.sum()) >= lo - slack and u * float(strict.sum()) <= hi + slack, (lo, hi, u, slack)


@pytest.mark.gpu
@pytest.mark.parametrize("V", [1000, 151936])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sample_kernel(V, dtype):
    torch.manual_seed(V)
    B = 12
    logits = (torch.randn(B, V, device="cuda") * 2.5).to(dtype)
    temps = torch.tensor([1.0, 0.7, 1.3, 0.0, 1.0, 1.0, 0.5, 1.0, 2.0, 1.0, 0.9, 1.0], device="cuda")
    ks = torch.tensor([0, 50, 0, 0, 1, 20, 0, 5, 0, 300, 0, V + 5], dtype=torch.int32, device="cuda")
    ps = torch.tensor([1.0, 1.0, 0.9, 1.0, 1.0, 0.8, 0.5, 1.0, 0.95, 0.99, 1.0, 0.0], device="cuda")
    mps = torch.tensor([0, 0, 0, 0, 0, 0, 0.05, 0.1, 0, 0, 0.3, 0], dtype=torch.float32, device="cuda")
    for trial in range(4):
        u = torch.rand(B, device="cuda", generator=torch.Generator(device="cuda").manual_seed(trial))
        got = ops.top_k_top_p_min_p_sample(logits, temps, ks, ps, mps, u).cpu()
        for b in range(B):
            tok = int(got[b])
            if float(temps[b]) <= 1e-6:
                assert tok == int(torch.argmax(logits[b].float())), b
                continue
            if int(ks[b]) == 1 or float(ps[b]) == 0.0:  # ties at the cut-off are all kept
                assert float(logits[b, tok]) == float(logits[b].max()), b
                continue
            _check_row(logits[b], float(temps[b]), int(ks[b]), float(ps[b]), float(mps[b]), float(u[b]), tok)
    ops.check_status()


@pytest.mark.gpu
def test_sample_kernel_distribution():
    """Empirical frequencies of many draws follow the filtered distribution."""
    probs = torch.tensor([0.4, 0.3, 0.15, 0.1, 0.05])
    logits = torch.log(probs).repeat(4096, 1).cuda()
    t, k, p = _params(4096, k=3, device="cuda")
    u = torch.rand(4096, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    got = ops.top_k_top_p_min_p_sample(logits, t, k, p, None, u)
    freq = torch.bincount(got.cpu(), minlength=5).float() / 4096
    want = torch.tensor([0.4, 0.3, 0.15, 0, 0]) / 0.85
    assert (freq - want).abs().max() < 0.03


@pytest.mark.gpu
def test_penalties_kernel():
    torch.manual_seed(0)
    B, V = 5, 3000
    logits = torch.randn(B, V, device="cuda")
    counts = torch.randint(0, 3, (B, V), device="cuda")
    pm = torch.rand(B, V, device="cuda") < 0.1
    f, pr, rp = torch.rand(B, device="cuda"), torch.rand(B, device="cuda"), 1 + torch.rand(B, device="cuda")
    got = ops.apply_penalties(logits.clone(), counts, pm, f, pr, rp)
    want = ref.apply_penalties(logits, counts, pm, f, pr, rp)
    torch.testing.assert_close(got, want, atol=1e-6, rtol=1e-6)

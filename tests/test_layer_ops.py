"""API-parity operator modules: stand-alone RoPE forms and the sampling operators."""
import torch

from mllm_b200.layers import rope, sampling
from mllm_b200.ops import reference as ref


def test_rope_forms_agree():
    torch.manual_seed(0)
    T, H, D = 7, 2, 16
    q, k = torch.randn(T, H, D), torch.randn(T, 1, D)
    indptr, offsets = torch.tensor([0, 3, 7]), torch.tensor([5, 0])
    pos = torch.tensor([5, 6, 7, 0, 1, 2, 3])
    a = rope.apply_rope(q, k, indptr, offsets, rope_theta=1e4)
    b = rope.apply_rope_pos_ids(q, k, pos, rope_theta=1e4)
    torch.testing.assert_close(a[0], b[0])
    cos, sin = ref.rope_cos_sin(pos, D, 1e4)
    torch.testing.assert_close(b[0], ref.apply_rope_neox(q, cos, sin))
    cache = torch.cat([cos, sin], -1)
    c = rope.apply_rope_with_cos_sin_cache(torch.arange(T), q.reshape(T, -1), k.reshape(T, -1), D,
                                           torch.cat(ref.rope_cos_sin(torch.arange(8), D, 1e4), -1))
    d = rope.apply_rope_pos_ids(q, k, torch.arange(T), rope_theta=1e4)
    torch.testing.assert_close(c[0].view(T, H, D), d[0])
    q2, k2 = q.clone(), k.clone()
    assert rope.apply_rope_pos_ids(q2, k2, pos, inplace=True, rope_theta=1e4) is None
    torch.testing.assert_close(q2, b[0])
    # interleaved pairing rotates (even, odd) pairs
    e = rope.apply_rope_pos_ids(q, k, pos, interleave=True, rope_theta=1e4)[0]
    x0, x1 = q[..., 0], q[..., 1]
    torch.testing.assert_close(e[..., 0], x0 * cos[:, :1] - x1 * sin[:, :1])
    # llama-3.1 scaling leaves the highest frequencies alone and divides the lowest by the scale
    f = rope._inv_freq(128, 5e5, "cpu", (8.0, 1.0, 4.0, 8192.0))
    g = rope._inv_freq(128, 5e5, "cpu")
    torch.testing.assert_close(f[0], g[0])
    torch.testing.assert_close(f[-1], g[-1] / 8.0)


def test_mrope_matches_reference_statement():
    torch.manual_seed(1)
    T, H, D = 6, 2, 128
    q, k = torch.randn(T, H, D), torch.randn(T, 1, D)
    pos3 = torch.randint(0, 50, (3, T))
    cache = torch.cat(ref.rope_cos_sin(torch.arange(64), D, 5e6), -1)
    for inter in (True, False):
        got = rope.apply_mrope(q, k, pos3, cache, [24, 20, 20], inter)[0]
        cos, sin = ref.mrope_cos_sin(pos3, D, 5e6, [24, 20, 20], inter)
        torch.testing.assert_close(got, ref.apply_rope_neox(q, cos, sin), atol=1e-5, rtol=1e-5)


def test_sampling_operators():
    torch.manual_seed(2)
    logits = torch.randn(64, 50) * 2
    probs = sampling.softmax(logits, temperature=0.7)
    torch.testing.assert_close(probs.sum(-1), torch.ones(64))
    rk = sampling.top_k_renorm_probs(probs, 5)
    assert ((rk > 0).sum(-1) == 5).all() and torch.allclose(rk.sum(-1), torch.ones(64))
    rp = sampling.top_p_renorm_probs(probs, 0.6)
    kept_mass = torch.where(rp > 0, probs, torch.zeros_like(probs)).sum(-1)
    assert (kept_mass >= 0.6 - 1e-5).all()
    ml = sampling.top_k_mask_logits(logits, 3)
    assert (torch.isfinite(ml).sum(-1) == 3).all()
    g = torch.Generator().manual_seed(0)
    ids = sampling.top_k_sampling_from_probs(probs, 5, generator=g)
    assert (rk.gather(1, ids.long().unsqueeze(1)) > 0).all()
    ids = sampling.top_p_sampling_from_probs(probs, 0.6, generator=g)
    assert (rp.gather(1, ids.long().unsqueeze(1)) > 0).all()
    ids = sampling.min_p_sampling_from_probs(probs, 0.2, generator=g)
    assert (probs.gather(1, ids.long().unsqueeze(1)).squeeze(1) >= 0.2 * probs.max(-1).values - 1e-6).all()
    ids = sampling.top_k_top_p_sampling_from_logits(logits, 8, 0.9, generator=g)
    assert (ml.shape[0] == ids.shape[0]) and ids.dtype == torch.int32
    a = sampling.sampling_from_logits(logits, seed=7)
    b = sampling.sampling_from_probs(torch.softmax(logits, -1), seed=7)
    assert torch.equal(a, b)


def test_chain_speculative_sampling():
    torch.manual_seed(3)
    B, n, V = 4, 3, 11
    target = torch.softmax(torch.randn(B, n + 1, V), -1)
    # identical draft and target distributions: every draft token is accepted, plus one bonus token
    draft = target[:, :n].clone()
    ids = torch.multinomial(draft.reshape(-1, V), 1).view(B, n)
    out, acc, emitted = sampling.chain_speculative_sampling(draft, ids, target, seed=1)
    assert torch.equal(out[:, :n], ids.int()) and (out[:, n] >= 0).all() and (emitted == n).all() and (acc == n).all()
    # a draft that always proposes a token the target gives zero mass: rejected at position 0
    tgt0 = target.clone()
    tgt0[:, :, 0] = 0
    tgt0 = tgt0 / tgt0.sum(-1, keepdim=True)
    bad = torch.zeros(B, n, V)
    bad[:, :, 0] = 1
    out, acc, emitted = sampling.chain_speculative_sampling(bad, torch.zeros(B, n, dtype=torch.long), tgt0, seed=1)
    assert (emitted == 0).all() and (out[:, 0] > 0).all() and (out[:, 1:] == -1).all()


def test_batched_decode_attention_equals_the_per_request_statement():
    import torch

    from mllm_b200.ops import reference as ref

    torch.manual_seed(0)
    B, Hq, Hkv, D, slots_n = 3, 4, 2, 24, 64
    kc, vc = torch.randn(slots_n, Hkv, D), torch.randn(slots_n, Hkv, D)
    rtt = torch.zeros(5, 20, dtype=torch.int32)
    seq = torch.tensor([7, 1, 13], dtype=torch.int32)
    req = torch.tensor([4, 0, 2], dtype=torch.int32)
    perm = torch.randperm(slots_n)[: int(seq.sum())].int()
    off = 0
    for b in range(B):
        rtt[req[b], : seq[b]] = perm[off: off + int(seq[b])]
        off += int(seq[b])
    q = torch.randn(B, Hq, D)
    want = ref.attention_decode(q, kc, vc, rtt, req, seq, D ** -0.5)
    got = ref.attention_decode_batched(q, kc, vc, rtt, req, seq, D ** -0.5, max_seq_len=16)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    out = torch.empty_like(q)
    ref.attention_decode_batched(q, kc, vc, rtt, req, seq, D ** -0.5, max_seq_len=13, out=out)
    torch.testing.assert_close(out, want, atol=1e-5, rtol=1e-5)


def test_sdpa_fallback_equals_the_softmax_statement():
    """Rectangular causal (queries after a cached prefix), square causal and unmasked cases, grouped heads."""
    import torch

    from mllm_b200.ops import reference as ref

    torch.manual_seed(1)
    for Tq, Tk, off in ((5, 12, 7), (9, 9, 0), (1, 6, None), (4, 4, None)):
        q, k, v = torch.randn(Tq, 4, 16), torch.randn(Tk, 2, 16), torch.randn(Tk, 2, 16)
        want = ref._attend(q, k, v, 0.25, off)
        got = ref._attend_sdpa(q, k, v, 0.25, off)
        torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_sdpa_prefill_fallback_equals_the_reference_prefill():
    import torch

    from mllm_b200.ops import reference as ref

    torch.manual_seed(2)
    Hq, Hkv, D = 4, 2, 16
    kc, vc = torch.randn(80, Hkv, D), torch.randn(80, Hkv, D)
    rtt = torch.zeros(4, 32, dtype=torch.int32)
    seq, pre = torch.tensor([9, 14], dtype=torch.int32), torch.tensor([0, 6], dtype=torch.int32)
    req = torch.tensor([3, 1], dtype=torch.int32)
    perm = torch.randperm(80).int()
    rtt[3, :9], rtt[1, :14] = perm[:9], perm[9:23]
    q = torch.randn(9 + 8, Hq, D)
    qs = torch.tensor([0, 9], dtype=torch.int32)
    want = ref.attention_prefill(q, kc, vc, rtt, req, seq, pre, qs, D ** -0.5)
    got = ref.attention_prefill_sdpa(q, kc, vc, rtt, req, seq, pre, qs, D ** -0.5)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    got = ref.attention_prefill_sdpa(q, kc, vc, rtt, req, seq, pre, qs, D ** -0.5, [9, 14], [0, 6])
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_window_and_logit_cap_agree_across_attention_paths():
    """Sliding window and soft-capping: the per-request statement, the batched decode form and the SDPA
    prefill form agree with a direct softmax evaluation."""
    import torch

    from mllm_b200.ops import reference as ref

    torch.manual_seed(3)
    Hq, Hkv, D, W, cap = 4, 2, 16, 5, 3.0
    kc, vc = torch.randn(64, Hkv, D), torch.randn(64, Hkv, D)
    rtt = torch.zeros(2, 32, dtype=torch.int32)
    rtt[0, :12], rtt[1, :20] = torch.arange(12).int(), torch.arange(20, 40).int()
    req, seq, pre = torch.tensor([0, 1], dtype=torch.int32), torch.tensor([12, 20], dtype=torch.int32), torch.tensor([0, 9], dtype=torch.int32)
    q = torch.randn(12 + 11, Hq, D)
    qs = torch.tensor([0, 12], dtype=torch.int32)
    scale = D ** -0.5
    # direct evaluation for request 1, query row 3 (absolute position 12): keys 8..12 visible
    want = ref.attention_prefill(q, kc, vc, rtt, req, seq, pre, qs, scale, window=W, logit_cap=cap)
    k1, v1 = kc[20:40].repeat_interleave(2, 1), vc[20:40].repeat_interleave(2, 1)
    s = torch.einsum("hd,khd->hk", q[12 + 3], k1) * scale
    s = cap * torch.tanh(s / cap)
    s[:, :8], s[:, 13:] = float("-inf"), float("-inf")
    torch.testing.assert_close(want[12 + 3], torch.einsum("hk,khd->hd", torch.softmax(s, -1), v1), atol=1e-5, rtol=1e-5)
    got = ref.attention_prefill_sdpa(q, kc, vc, rtt, req, seq, pre, qs, scale, window=W)
    torch.testing.assert_close(got, ref.attention_prefill(q, kc, vc, rtt, req, seq, pre, qs, scale, window=W), atol=1e-5, rtol=1e-5)
    qd = torch.randn(2, Hq, D)
    a = ref.attention_decode(qd, kc, vc, rtt, req, seq, scale, window=W, logit_cap=cap)
    b = ref.attention_decode_batched(qd, kc, vc, rtt, req, seq, scale, 24, window=W, logit_cap=cap)
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)
    assert not torch.allclose(a, ref.attention_decode(qd, kc, vc, rtt, req, seq, scale), atol=1e-3)


def test_create_kv_indices_matches_a_python_loop():
    import torch

    from mllm_b200 import ops

    torch.manual_seed(4)
    rtt = torch.randint(0, 1000, (6, 40), dtype=torch.int32)
    req = torch.tensor([4, 0, 5], dtype=torch.int32)
    lens = torch.tensor([7, 0, 19], dtype=torch.int32)
    start = torch.tensor([2, 0, 11], dtype=torch.int32)
    indptr, idx = ops.create_kv_indices(rtt, req, lens, start)
    want = []
    for b in range(3):
        want += rtt[req[b], start[b]: start[b] + lens[b]].tolist()
    assert indptr.tolist() == [0, 7, 7, 26] and idx.tolist() == want and idx.dtype == torch.int32
    indptr2, idx2 = ops.create_kv_indices(rtt, req, lens, max_len=32)
    assert idx2.tolist() == rtt[4, :7].tolist() + rtt[5, :19].tolist()

"""Sampling operators under the names the reference exposes (pymllm/layers/sampling.py:56-760):
temperature softmax, sampling from probabilities / logits, top-p / top-k / min-p sampling,
renormalisation, logit masking and chain speculative sampling.

The filtered samplers run on the sort-free CUDA kernel (`ops.top_k_top_p_min_p_sample`): probabilities
are turned into logits (``log p``, temperature 1) and the uniform numbers come from the caller's
generator, so a seeded generator reproduces a run.  The remaining operators are short PyTorch
expressions; they are not on the serving hot path (the model runner calls the fused kernel directly).
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from .. import ops

Scalar = Union[torch.Tensor, float, int]


def _per_row(value: Scalar, batch: int, device, dtype=torch.float32) -> torch.Tensor:
    if isinstance(value, torch.Tensor):
        return value.to(device=device, dtype=dtype).reshape(-1).expand(batch).contiguous()
    return torch.full((batch,), value, device=device, dtype=dtype)


def _rows(data: torch.Tensor, indices: Optional[torch.Tensor]) -> torch.Tensor:
    return data if indices is None else data[indices.long()]


def _uniform(batch: int, device, generator: Optional[torch.Generator], seed: Optional[int]) -> torch.Tensor:
    if generator is None and seed is not None:
        generator = torch.Generator(device=device)
        generator.manual_seed(int(seed))
    return torch.rand(batch, device=device, generator=generator)


def softmax(logits: torch.Tensor, temperature: Optional[Scalar] = None, enable_pdl: Optional[bool] = None) -> torch.Tensor:
    """Temperature softmax; a temperature below 1e-6 means "no scaling" (greedy rows are handled by argmax)."""
    if temperature is not None:
        if isinstance(temperature, torch.Tensor):
            logits = logits / temperature.clamp(min=1e-6).reshape(-1, 1).to(logits.dtype)
        elif temperature >= 1e-6:
            logits = logits / temperature
    return torch.softmax(logits.float(), dim=-1)


def _sample(logits: torch.Tensor, top_k, top_p, min_p, generator, seed) -> torch.Tensor:
    b, dev = logits.shape[0], logits.device
    return ops.top_k_top_p_min_p_sample(
        logits, torch.ones(b, device=dev), _per_row(top_k, b, dev, torch.int32), _per_row(top_p, b, dev),
        None if min_p is None else _per_row(min_p, b, dev), _uniform(b, dev, generator, seed)).to(torch.int32)


def _log_probs(probs: torch.Tensor) -> torch.Tensor:
    return torch.log(probs.float().clamp_min(0)).contiguous()  # log 0 = -inf: never sampled


def sampling_from_probs(probs, indices=None, deterministic: bool = True, generator=None, check_nan: bool = False,
                        seed: Optional[int] = None, offset: Optional[int] = None) -> torch.Tensor:
    probs = _rows(probs, indices)
    if check_nan and torch.isnan(probs).any():
        raise ValueError("NaN in probabilities")
    return _sample(_log_probs(probs), 0, 1.0, None, generator, seed)


def sampling_from_logits(logits, indices=None, deterministic: bool = True, generator=None, check_nan: bool = False,
                         seed: Optional[int] = None, offset: Optional[int] = None) -> torch.Tensor:
    logits = _rows(logits, indices)
    if check_nan and torch.isnan(logits).any():
        raise ValueError("NaN in logits")
    return _sample(logits.contiguous(), 0, 1.0, None, generator, seed)


def top_p_sampling_from_probs(probs, top_p: Scalar, indices=None, deterministic: bool = True, generator=None,
                              check_nan: bool = False, seed=None, offset=None) -> torch.Tensor:
    return _sample(_log_probs(_rows(probs, indices)), 0, top_p, None, generator, seed)


def top_k_sampling_from_probs(probs, top_k: Scalar, indices=None, deterministic: bool = True, generator=None,
                              check_nan: bool = False, seed=None, offset=None) -> torch.Tensor:
    return _sample(_log_probs(_rows(probs, indices)), top_k, 1.0, None, generator, seed)


def min_p_sampling_from_probs(probs, min_p: Scalar, indices=None, deterministic: bool = True, generator=None,
                              check_nan: bool = False, seed=None, offset=None) -> torch.Tensor:
    return _sample(_log_probs(_rows(probs, indices)), 0, 1.0, min_p, generator, seed)


def top_k_top_p_sampling_from_logits(logits, top_k: Scalar, top_p: Scalar, indices=None, filter_apply_order: str = "top_k_first",
                                     deterministic: bool = True, generator=None, check_nan: bool = False, seed=None,
                                     offset=None) -> torch.Tensor:
    """Both filters are cut-offs on the same distribution ("joint"); with ``top_k_first`` the top-p mass is
    taken over the renormalised top-k set, as the reference does."""
    logits = _rows(logits, indices)
    if filter_apply_order == "top_k_first":
        logits = top_k_mask_logits(logits, top_k)
        return _sample(logits.contiguous(), 0, top_p, None, generator, seed)
    return _sample(logits.contiguous(), top_k, top_p, None, generator, seed)


def top_k_top_p_sampling_from_probs(probs, top_k: Scalar, top_p: Scalar, indices=None, filter_apply_order: str = "top_k_first",
                                    deterministic: bool = True, generator=None, check_nan: bool = False, seed=None,
                                    offset=None) -> torch.Tensor:
    return top_k_top_p_sampling_from_logits(_log_probs(_rows(probs, indices)), top_k, top_p, None, filter_apply_order,
                                            deterministic, generator, check_nan, seed, offset)


def top_p_renorm_probs(probs: torch.Tensor, top_p: Scalar) -> torch.Tensor:
    """Keep the smallest descending prefix whose mass reaches ``top_p``; renormalise."""
    p = probs.float()
    tp = _per_row(top_p, p.shape[0], p.device).unsqueeze(-1)
    sp, si = torch.sort(p, dim=-1, descending=True)
    before = torch.cumsum(sp, -1) - sp
    sp = torch.where(before < tp, sp, torch.zeros_like(sp))
    out = torch.zeros_like(p).scatter_(-1, si, sp)
    return out / out.sum(-1, keepdim=True)


def top_k_renorm_probs(probs: torch.Tensor, top_k: Scalar) -> torch.Tensor:
    p = probs.float()
    k = _per_row(top_k, p.shape[0], p.device, torch.int64).clamp(1, p.shape[-1])
    sp = torch.sort(p, dim=-1, descending=True).values
    thr = sp.gather(-1, (k - 1).unsqueeze(-1))
    out = torch.where(p >= thr, p, torch.zeros_like(p))
    return out / out.sum(-1, keepdim=True)


def top_k_mask_logits(logits: torch.Tensor, top_k: Scalar) -> torch.Tensor:
    """Logits outside the per-row top-k set to -inf (ties at the cut-off are kept)."""
    k = _per_row(top_k, logits.shape[0], logits.device, torch.int64)
    k = torch.where(k <= 0, torch.full_like(k, logits.shape[-1]), k).clamp(max=logits.shape[-1])
    sl = torch.sort(logits.float(), dim=-1, descending=True).values
    thr = sl.gather(-1, (k - 1).unsqueeze(-1))
    return torch.where(logits.float() >= thr, logits.float(), torch.full_like(logits, float("-inf"), dtype=torch.float32))


def chain_speculative_sampling(draft_probs: torch.Tensor, draft_token_ids: torch.Tensor, target_probs: torch.Tensor,
                               maybe_output_accepted_token_num: Optional[torch.Tensor] = None,
                               maybe_output_emitted_draft_token_num: Optional[torch.Tensor] = None,
                               deterministic: bool = True, generator: Optional[torch.Generator] = None,
                               seed: Optional[int] = None, offset: Optional[int] = None
                               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Accept draft token i with probability ``min(1, p_target / p_draft)``; at the first rejection sample
    from ``normalise(max(p_target - p_draft, 0))``; if all are accepted sample the bonus token from the last
    target distribution.  Returns (tokens [B, n+1] padded with -1, accepted counts, emitted counts)."""
    B, n, V = draft_probs.shape
    dev = draft_probs.device
    if generator is None and seed is not None:
        generator = torch.Generator(device=dev)
        generator.manual_seed(int(seed))
    u = torch.rand(B, n, device=dev, generator=generator)
    u_final = torch.rand(B, device=dev, generator=generator)
    ids = draft_token_ids.long()
    p_d = draft_probs.float().gather(-1, ids.unsqueeze(-1)).squeeze(-1)
    p_t = target_probs.float()[:, :n].gather(-1, ids.unsqueeze(-1)).squeeze(-1)
    ok = u * p_d <= p_t                                               # accept test per position
    accepted_all = ok.long().sum(-1)                                  # independent acceptances (statistic)
    first_rej = torch.where(ok.all(-1), torch.full((B,), n, device=dev), (~ok).float().argmax(-1))
    out = torch.full((B, n + 1), -1, dtype=torch.int32, device=dev)
    pos = torch.arange(n, device=dev).unsqueeze(0)
    out[:, :n] = torch.where(pos < first_rej.unsqueeze(-1), draft_token_ids.to(torch.int32), out[:, :n])
    # distribution of the extra token
    rows = torch.arange(B, device=dev)
    tgt = target_probs.float()[rows, first_rej]
    drf = torch.where((first_rej < n).unsqueeze(-1), draft_probs.float()[rows, first_rej.clamp(max=n - 1)], torch.zeros_like(tgt))
    resid = (tgt - drf).clamp_min(0)
    resid = torch.where(resid.sum(-1, keepdim=True) > 0, resid, tgt)
    cdf = torch.cumsum(resid / resid.sum(-1, keepdim=True), -1)
    extra = (cdf <= u_final.unsqueeze(-1)).long().sum(-1).clamp(max=V - 1)
    out[rows, first_rej] = extra.to(torch.int32)
    if maybe_output_accepted_token_num is not None:
        maybe_output_accepted_token_num += accepted_all.to(maybe_output_accepted_token_num.dtype)
        accepted_all = maybe_output_accepted_token_num
    if maybe_output_emitted_draft_token_num is not None:
        maybe_output_emitted_draft_token_num += first_rej.to(maybe_output_emitted_draft_token_num.dtype)
        first_rej = maybe_output_emitted_draft_token_num
    return out, accepted_all, first_rej

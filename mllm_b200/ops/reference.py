"""Plain-PyTorch statement of every op in :mod:`mllm_b200.ops`.

These functions are the numerical contract of the CUDA kernels: each kernel's
test compares against the function of the same name evaluated in fp32.  They
also run the whole engine on a machine without a GPU (CPU tests, the fp32
oracle of the Qwen3 model).  They are never used for tensors that live on a
GPU unless ``MLLM_B200_FORCE_TORCH=1`` is set for A/B comparisons.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def _f32(x: torch.Tensor) -> torch.Tensor:
    return x.float()


# --------------------------------------------------------------------------
# normalisation / activation / embedding
# --------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    xf = _f32(x)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * _f32(weight)
    y = y.to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """In place: ``residual += x`` (rounded to the storage dtype), ``x = rmsnorm(residual) * weight``."""
    s = (_f32(x) + _f32(residual)).to(residual.dtype)
    residual.copy_(s)
    x.copy_(rmsnorm(s, weight, eps))


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return F.layer_norm(_f32(x), (x.shape[-1],), _f32(weight), None if bias is None else _f32(bias), eps).to(x.dtype)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.silu(_f32(x[..., :d])) * _f32(x[..., d:])).to(x.dtype)


def gelu_tanh_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.gelu(_f32(x[..., :d]), approximate="tanh") * _f32(x[..., d:])).to(x.dtype)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(_f32(x), approximate="tanh").to(x.dtype)


def gelu_erf(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(_f32(x)).to(x.dtype)


def vision_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """2-D rotary embedding of the vision tower: x [T, H, D], cos/sin [T, D/2] (first quarter of the
    frequencies from the row position, second from the column position); pairs (i, i + D/2)
    (pymllm/models/qwen3_vl.py:118-167)."""
    xf = _f32(x)
    half = x.shape[-1] // 2
    c, s = _f32(cos).unsqueeze(1), _f32(sin).unsqueeze(1)
    x1, x2 = xf[..., :half], xf[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def vision_pos_embed_add(x: torch.Tensor, table: torch.Tensor, idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x + sum_i w[i] * table[idx[i]]`` over the four bilinear corners (pymllm/models/qwen3_vl.py:456-491)."""
    pe = (_f32(table)[idx] * w.float().unsqueeze(-1)).sum(0)
    return (_f32(x) + pe).to(x.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return table[ids.long()]


# --------------------------------------------------------------------------
# GEMMs
# --------------------------------------------------------------------------
def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """``x @ weight.T (+ bias) (+ residual)`` with fp32 accumulation, one rounding at the end."""
    y = _f32(x) @ _f32(weight).t()
    if bias is not None:
        y = y + _f32(bias)
    if residual is not None:
        y = y + _f32(residual)
    return y.to(out_dtype or x.dtype)


def deinterleave_gate_up(y: torch.Tensor, block: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split the columns of a ``[.., 2I]`` tensor whose columns alternate
    ``block`` gate features, ``block`` up features, ... into (gate, up)."""
    lead = y.shape[:-1]
    v = y.reshape(*lead, -1, 2, block)
    return v[..., 0, :].reshape(*lead, -1), v[..., 1, :].reshape(*lead, -1)


def interleave_gate_up(w: torch.Tensor, block: int) -> torch.Tensor:
    """Rows ``[gate(I) ; up(I)]`` -> rows alternating ``block`` gate, ``block`` up."""
    i = w.shape[0] // 2
    g = w[:i].reshape(i // block, 1, block, *w.shape[1:])
    u = w[i:].reshape(i // block, 1, block, *w.shape[1:])
    return torch.cat([g, u], dim=1).reshape(w.shape)


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor, block: int = 0) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)``; ``block`` = row interleave of ``weight`` (0: ``[gate ; up]``)."""
    y = _f32(x) @ _f32(weight).t()
    if block:
        g, u = deinterleave_gate_up(y, block)
    else:
        d = y.shape[-1] // 2
        g, u = y[..., :d], y[..., d:]
    return (F.silu(g) * u).to(x.dtype)


def per_token_quant_int8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-row int8: ``scale = absmax/127``, ``q = round(x/scale)``."""
    xf = _f32(x)
    absmax = xf.abs().amax(-1, keepdim=True).clamp_min(1e-10)
    scale = absmax / 127.0
    q = torch.round(xf / scale).clamp(-128, 127).to(torch.int8)
    return q, scale.float()


def int8_scaled_mm(
    a_q: torch.Tensor, w_q: torch.Tensor, a_scale: torch.Tensor, w_scale: torch.Tensor,
    out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``(a_q @ w_q.T) * a_scale[M,1] * w_scale[N]`` with exact int32 accumulation."""
    acc = (a_q.to(torch.int32).cpu() @ w_q.to(torch.int32).cpu().t()).to(a_q.device) if a_q.is_cuda else (
        a_q.to(torch.int32) @ w_q.to(torch.int32).t())
    y = acc.float() * a_scale.reshape(-1, 1).float() * w_scale.reshape(1, -1).float()
    if bias is not None:
        y = y + _f32(bias)
    return y.to(out_dtype)


def unpack_int4_rows(packed: torch.Tensor) -> torch.Tensor:
    """int32 ``[N, K/8]`` (nibble i of word j = element 8j+i) -> uint8-valued ``[N, K]`` in 0..15."""
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    return ((packed.unsqueeze(-1) >> shifts) & 0xF).reshape(packed.shape[0], -1)


def dequant_w4(qweight: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor], group: int) -> torch.Tensor:
    """``qweight`` int32 ``[N, K/8]``, ``scales`` ``[N, K/g]``, ``zeros`` uint8-valued ``[N, K/g]`` or
    None (symmetric, zero point 8) -> fp32 ``[N, K]``."""
    q = unpack_int4_rows(qweight).float()
    s = scales.float().repeat_interleave(group, dim=1)
    z = 8.0 if zeros is None else zeros.float().repeat_interleave(group, dim=1)
    return (q - z) * s


def w4a16_gemm(x, qweight, scales, zeros, group: int, bias=None) -> torch.Tensor:
    y = _f32(x) @ dequant_w4(qweight, scales, zeros, group).t()
    if bias is not None:
        y = y + _f32(bias)
    return y.to(x.dtype)


# --------------------------------------------------------------------------
# rotary embedding, QK-norm, cache write
# --------------------------------------------------------------------------
def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, rotary_dim: Optional[int] = None,
                 inv_freq: Optional[torch.Tensor] = None):
    rd = rotary_dim or head_dim
    inv = inv_freq.to(positions.device) if inv_freq is not None else \
        1.0 / (theta ** (torch.arange(0, rd, 2, device=positions.device, dtype=torch.float32) / rd))
    ang = positions.float().unsqueeze(-1) * inv  # [..., rd/2]
    return ang.cos(), ang.sin()


def apply_rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, H, D] fp32; cos/sin: [T, rd/2]; rotates the first ``rd`` features (half-split pairing)."""
    half = cos.shape[-1]
    x1, x2, rest = x[..., :half], x[..., half : 2 * half], x[..., 2 * half :]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


def mrope_cos_sin(positions3: torch.Tensor, head_dim: int, theta: float, sections, interleaved: bool):
    """positions3: [3, T] (t, h, w).  Returns cos/sin [T, D/2] whose frequency
    index i takes its position from axis ``a(i)``: consecutive sections
    ``[t]*s0 + [h]*s1 + [w]*s2`` or, when ``interleaved``, ``a(i) = i % 3`` for
    ``i < 3*s1`` / ``3*s2`` (h, w) and t elsewhere (pymllm/layers/rope.py:320-408)."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions3.device, dtype=torch.float32) / head_dim))
    ang = positions3.float().unsqueeze(-1) * inv  # [3, T, half]
    axis = torch.zeros(half, dtype=torch.long, device=positions3.device)
    if interleaved:
        idx = torch.arange(half, device=positions3.device)
        axis[(idx % 3 == 1) & (idx < 3 * sections[1])] = 1
        axis[(idx % 3 == 2) & (idx < 3 * sections[2])] = 2
    else:
        axis[sections[0] : sections[0] + sections[1]] = 1
        axis[sections[0] + sections[1] : sections[0] + sections[1] + sections[2]] = 2
    sel = ang.permute(1, 2, 0).gather(-1, axis.view(1, half, 1).expand(ang.shape[1], half, 1)).squeeze(-1)
    return sel.cos(), sel.sin()


def qk_norm_rope_kv_write(
    qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
    positions: torch.Tensor, cache_loc: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
    num_q_heads: int, num_kv_heads: int, head_dim: int, theta: float, eps: float,
    mrope_sections=None, mrope_interleaved: bool = False, inv_freq: Optional[torch.Tensor] = None,
) -> None:
    """In place on ``qkv`` ``[T, (Hq+2Hkv)*D]``: per-head RMSNorm of q and k (if weights
    given), NeoX RoPE at ``positions`` (``[T]``, or ``[3,T]`` with ``mrope_sections``); then
    ``k_cache[cache_loc] = k`` (normed, rotated) and ``v_cache[cache_loc] = v``."""
    T = qkv.shape[0]
    qd, kd = num_q_heads * head_dim, num_kv_heads * head_dim
    q = _f32(qkv[:, :qd]).reshape(T, num_q_heads, head_dim)
    k = _f32(qkv[:, qd : qd + kd]).reshape(T, num_kv_heads, head_dim)
    v = qkv[:, qd + kd :].reshape(T, num_kv_heads, head_dim)
    if q_weight is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * _f32(q_weight)
        q = q.to(qkv.dtype).float()
    if k_weight is not None:
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * _f32(k_weight)
        k = k.to(qkv.dtype).float()
    if mrope_sections is not None:
        cos, sin = mrope_cos_sin(positions, head_dim, theta, mrope_sections, mrope_interleaved)
    else:
        cos, sin = rope_cos_sin(positions, head_dim, theta, inv_freq=inv_freq)
    q = apply_rope_neox(q, cos, sin).to(qkv.dtype)
    k = apply_rope_neox(k, cos, sin).to(qkv.dtype)
    qkv[:, :qd] = q.reshape(T, qd)
    qkv[:, qd : qd + kd] = k.reshape(T, kd)
    loc = cache_loc.long()
    k_cache[loc] = k.to(k_cache.dtype)
    v_cache[loc] = v.to(v_cache.dtype)


def kv_write(k, v, loc, k_cache, v_cache) -> None:
    """k, v: [T, Hkv * D] or [T, Hkv, D] rows written to the cache slots ``loc``."""
    k_cache[loc.long()] = k.reshape(k.shape[0], *k_cache.shape[1:]).to(k_cache.dtype)
    v_cache[loc.long()] = v.reshape(v.shape[0], *v_cache.shape[1:]).to(v_cache.dtype)


def create_kv_indices(req_to_token: torch.Tensor, req_pool_indices: torch.Tensor, seq_lens: torch.Tensor,
                      kv_start: Optional[torch.Tensor] = None, max_len: Optional[int] = None):
    """Flat KV index list of a batch, as paged-attention libraries want it (role of mllm-kernel's
    ``create_kv_indices``): ``kv_indices[kv_indptr[b] + j] = req_to_token[req_pool_indices[b], kv_start[b] + j]``
    for ``j < seq_lens[b]``.  Returns ``(kv_indptr int32 [B + 1], kv_indices int32 [sum(seq_lens)])``.  The
    attention kernels of this package read ``req_to_token`` directly and do not need it."""
    lens = seq_lens.to(torch.int64)
    B = lens.numel()
    indptr = torch.zeros(B + 1, dtype=torch.int32, device=lens.device)
    indptr[1:] = torch.cumsum(lens, 0).to(torch.int32)
    width = int(max_len if max_len is not None else (int(lens.max()) if B else 0))
    j = torch.arange(width, device=lens.device).unsqueeze(0)
    start = kv_start.to(torch.int64).view(-1, 1) if kv_start is not None else 0
    cols = (j + start).clamp_(max=req_to_token.shape[1] - 1)
    rows = req_to_token[req_pool_indices.long().view(-1, 1), cols]
    return indptr, rows[j < lens.view(-1, 1)].to(torch.int32)


# --------------------------------------------------------------------------
# attention over the slot-indexed KV pool
# --------------------------------------------------------------------------
def _attend(q, k, v, scale, causal_offset: Optional[int], window: Optional[int] = None, logit_cap: float = 0.0):
    """q [Tq,Hq,D] k,v [Tk,Hkv,D] fp32 -> [Tq,Hq,D]; key j visible to query i iff j <= i + causal_offset and,
    with a sliding ``window``, j > i + causal_offset - window (the last ``window`` keys, the query's own
    included).  ``logit_cap`` > 0 soft-caps the scaled scores: ``cap * tanh(s / cap)``."""
    Hq, Hkv = q.shape[1], k.shape[1]
    g = Hq // Hkv
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    if logit_cap and logit_cap > 0:
        s = logit_cap * torch.tanh(s / logit_cap)
    if causal_offset is not None or window:
        off = causal_offset if causal_offset is not None else k.shape[0] - q.shape[0]
        i = torch.arange(q.shape[0], device=q.device).unsqueeze(-1)
        j = torch.arange(k.shape[0], device=q.device).unsqueeze(0)
        hidden = j > i + off if causal_offset is not None else torch.zeros_like(j > i)
        if window:
            hidden = hidden | (j <= i + off - int(window))
        s = s.masked_fill(hidden, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vv)


def _attend_sdpa(q, k, v, scale, causal_offset: Optional[int], window: Optional[int] = None):
    """:func:`_attend` through ``scaled_dot_product_attention`` in the tensors' own dtype (no fp32 score
    matrix): the fallback used on GPUs for head sizes without a kernel.  q [Tq,Hq,D], k / v [Tk,Hkv,D]."""
    import torch.nn.functional as F

    Tq, Tk = q.shape[0], k.shape[0]
    qh, kh, vh = q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0)
    mask, causal = None, False
    if causal_offset is not None:
        if causal_offset == 0 and Tq == Tk and not window:
            causal = True
        else:
            i = torch.arange(Tq, device=q.device).unsqueeze(-1)
            j = torch.arange(Tk, device=q.device).unsqueeze(0)
            mask = j <= i + causal_offset
            if window:
                mask = mask & (j > i + causal_offset - int(window))
    o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, is_causal=causal, scale=scale,
                                       enable_gqa=q.shape[1] != k.shape[1])
    return o.squeeze(0).transpose(0, 1)


def attention_prefill(
    q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, req_to_token: torch.Tensor,
    req_pool_indices: torch.Tensor, seq_lens: torch.Tensor, prefix_lens: torch.Tensor,
    q_start_loc: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None, max_q_len: int = 0,
    window: Optional[int] = None, logit_cap: float = 0.0,
) -> torch.Tensor:
    """Causal attention of each request's new tokens over its cached prefix plus itself.

    Request ``b`` owns query rows ``q_start_loc[b] .. +seq_lens[b]-prefix_lens[b]``; its keys
    are the slots ``req_to_token[req_pool_indices[b], :seq_lens[b]]``; query ``i`` sees keys
    ``0 .. prefix_lens[b]+i``."""
    out = torch.empty_like(q) if out is None else out
    for b in range(req_pool_indices.numel()):
        sl, pl, qs = int(seq_lens[b]), int(prefix_lens[b]), int(q_start_loc[b])
        n = sl - pl
        slots = req_to_token[int(req_pool_indices[b]), :sl].long()
        o = _attend(_f32(q[qs : qs + n]), _f32(k_cache[slots]), _f32(v_cache[slots]), scale, pl, window, logit_cap)
        out[qs : qs + n] = o.to(out.dtype)
    return out


def attention_prefill_sdpa(q, k_cache, v_cache, req_to_token, req_pool_indices, seq_lens, prefix_lens, q_start_loc,
                           scale: float, seq_lens_cpu=None, prefix_lens_cpu=None, window: Optional[int] = None) -> torch.Tensor:
    """:func:`attention_prefill` with ``scaled_dot_product_attention`` per request in the activation dtype —
    not a numerical reference but the serving fallback on GPUs for head sizes without a kernel.  The host
    copies of the lengths avoid device read-backs."""
    out = torch.empty_like(q)
    sls = seq_lens_cpu if seq_lens_cpu is not None else seq_lens.tolist()
    pls = prefix_lens_cpu if prefix_lens_cpu is not None else prefix_lens.tolist()
    qs = 0
    pools = req_pool_indices.long()
    for b, (sl, pl) in enumerate(zip(sls, pls)):
        n = int(sl) - int(pl)
        slots = req_to_token[pools[b], : int(sl)].long()
        out[qs : qs + n] = _attend_sdpa(q[qs : qs + n], k_cache[slots].to(q.dtype), v_cache[slots].to(q.dtype), scale, int(pl), window)
        qs += n
    return out


def attention_decode(
    q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, req_to_token: torch.Tensor,
    req_pool_indices: torch.Tensor, seq_lens: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None,
    window: Optional[int] = None, logit_cap: float = 0.0,
) -> torch.Tensor:
    """One query token per request over ``req_to_token[req, :seq_len]`` (the new token's K/V included)."""
    out = torch.empty_like(q) if out is None else out
    for b in range(req_pool_indices.numel()):
        sl = int(seq_lens[b])
        slots = req_to_token[int(req_pool_indices[b]), :sl].long()
        o = _attend(_f32(q[b : b + 1]), _f32(k_cache[slots]), _f32(v_cache[slots]), scale, None, window, logit_cap)
        out[b] = o[0].to(out.dtype)
    return out


def attention_decode_batched(
    q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, req_to_token: torch.Tensor,
    req_pool_indices: torch.Tensor, seq_lens: torch.Tensor, scale: float, max_seq_len: int,
    out: Optional[torch.Tensor] = None, window: Optional[int] = None, logit_cap: float = 0.0,
) -> torch.Tensor:
    """:func:`attention_decode` for the whole batch at once: keys are gathered up to ``max_seq_len`` (a host
    bound on ``seq_lens``) and the tail of every request is masked, so nothing is read back from the device.
    Used on GPUs for head sizes the decode kernel does not cover."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    S = int(max_seq_len)
    slots = req_to_token[req_pool_indices.long(), :S].long()                  # [B, S]
    k = _f32(k_cache[slots])                                                  # [B, S, Hkv, D]
    v = _f32(v_cache[slots])
    qg = _f32(q).view(B, Hkv, Hq // Hkv, D)
    s = torch.einsum("bhgd,bshd->bhgs", qg, k) * scale
    if logit_cap and logit_cap > 0:
        s = logit_cap * torch.tanh(s / logit_cap)
    pos = torch.arange(S, device=q.device).unsqueeze(0)
    valid = pos < seq_lens.view(-1, 1)
    if window:
        valid = valid & (pos >= seq_lens.view(-1, 1) - int(window))
    s = s.masked_fill(~valid.view(B, 1, 1, S), float("-inf"))
    o = torch.einsum("bhgs,bshd->bhgd", torch.softmax(s, dim=-1), v).reshape(B, Hq, D)
    if out is None:
        return o.to(q.dtype)
    out.copy_(o)
    return out


def attention_varlen_bidirectional(q, k, v, cu_seqlens, scale) -> torch.Tensor:
    """Full (non-causal) attention inside each segment ``cu_seqlens[i]..cu_seqlens[i+1]``; q,k,v [T,H,D]."""
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for a, b in zip(cu[:-1], cu[1:]):
        out[a:b] = _attend(_f32(q[a:b]), _f32(k[a:b]), _f32(v[a:b]), scale, None).to(q.dtype)
    return out


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> torch.Tensor:
    return torch.argmax(logits.float(), dim=-1)


def apply_penalties(logits, output_counts, prompt_mask, frequency_penalty, presence_penalty, repetition_penalty):
    """OpenAI-style frequency/presence penalties on generated-token counts and HF-style
    repetition penalty on tokens seen in prompt or output.  All per-request vectors are [B]."""
    lf = logits.float()
    seen_out = output_counts > 0
    lf = lf - frequency_penalty.view(-1, 1) * output_counts.float() - presence_penalty.view(-1, 1) * seen_out.float()
    seen = seen_out | prompt_mask
    rp = repetition_penalty.view(-1, 1)
    lf = torch.where(seen, torch.where(lf > 0, lf / rp, lf * rp), lf)
    return lf


def top_k_top_p_min_p_sample(
    logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
    min_p: Optional[torch.Tensor], uniform: torch.Tensor,
) -> torch.Tensor:
    """Sample one id per row.  ``temperature <= 1e-6`` rows are greedy; ``top_k <= 0`` disables top-k.

    With ``e = exp((logits - max) / T)`` every filter is a cut-off on ``e`` (values equal to the cut-off
    are all kept): top-k keeps ``e >= k-th largest``; top-p keeps the values whose strictly-larger mass
    is below ``top_p * sum(e)``; min-p keeps ``e >= min_p`` (the largest ``e`` is 1).  ``uniform`` [B]
    in [0,1) drives inverse-CDF sampling over the kept set in token-id order: the first id whose running
    kept mass exceeds ``u * kept_mass``."""
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.long, device=logits.device)
    for b in range(B):
        t = float(temperature[b])
        row = logits[b].float()
        if t <= 1e-6:
            out[b] = torch.argmax(row)
            continue
        e = torch.exp((row - row.max()) / t).double()
        tau = 0.0
        k = int(top_k[b])
        se = torch.sort(e, descending=True).values
        if 0 < k < V:
            tau = max(tau, float(se[k - 1]))
        tp = float(top_p[b])
        if tp < 1.0:
            before = torch.cumsum(se, 0) - se
            n = int((before < max(tp * float(se.sum()), 1e-30)).sum())
            tau = max(tau, float(se[max(n, 1) - 1]))
        if min_p is not None and float(min_p[b]) > 0:
            tau = max(tau, min(float(min_p[b]), 1.0))
        kept = torch.where(e >= tau, e, torch.zeros_like(e))
        cdf = torch.cumsum(kept, 0)
        target = float(uniform[b]) * float(cdf[-1])
        idx = int((cdf > target).nonzero()[0]) if bool((cdf > target).any()) else int((kept > 0).nonzero()[-1])
        out[b] = idx
    return out


# --------------------------------------------------------------------------
# mixture of experts
# --------------------------------------------------------------------------
def moe_router_topk(hidden: torch.Tensor, gate_weight: torch.Tensor, top_k: int, renormalize: bool = True):
    """fp32 ``softmax(hidden @ gate_weight.T)`` over all experts -> top-k (sorted by weight) ->
    optional renormalisation of the k weights (mllm/models/qwen3_moe/modeling_qwen3_moe_fa2.hpp:121-138).
    Returns (weights fp32 [T, k], expert ids int32 [T, k])."""
    logits = _f32(hidden) @ _f32(gate_weight).t()
    scores = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(scores, top_k, dim=-1, sorted=True)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, idx.to(torch.int32)


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
                expert_offset: int = 0, swiglu_block: int = 0) -> torch.Tensor:
    """Sum over the k routed experts of ``w * down_e(silu(gate_e(x)) * up_e(x))``.

    ``w13`` [E_local, 2I, H] (rows ``[gate ; up]``, or interleaved in ``swiglu_block`` rows), ``w2``
    [E_local, H, I]; expert ids outside ``[expert_offset, expert_offset + E_local)`` contribute
    nothing (they live on another expert-parallel rank)."""
    T, H = x.shape
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    E = w13.shape[0]
    for e in range(E):
        tok, slot = (topk_ids == (e + expert_offset)).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = linear_swiglu(x[tok], w13[e], swiglu_block)
        y = linear(h, w2[e], out_dtype=torch.float32)
        out.index_add_(0, tok, y * topk_w[tok, slot].unsqueeze(-1).float())
    return out.to(x.dtype)


# --------------------------------------------------------------------------
# gated delta net (linear attention of the Qwen3.5 hybrid models)
# --------------------------------------------------------------------------
def rmsnorm_gated(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``weight * round(rmsnorm(x)) * silu(gate)`` over the last dimension (norm before gate)."""
    xf = _f32(x)
    n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return (_f32(weight) * _f32(n) * F.silu(_f32(gate))).to(x.dtype)


def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, conv_state: torch.Tensor, state_indices: torch.Tensor,
                       seq_lens, has_state) -> torch.Tensor:
    """Depth-wise causal convolution (kernel K) + SiLU over ragged sequences.

    ``x`` [T, C] holds the new tokens of every request back to back (``seq_lens`` each); ``weight`` [C, K];
    ``conv_state`` [slots, C, K-1] keeps the last K-1 inputs of each request (row ``state_indices[b]``),
    read when ``has_state[b]`` (a continuation) and always written back."""
    K = weight.shape[1]
    out = torch.empty_like(x)
    off = 0
    for b, n in enumerate(list(seq_lens)):
        n = int(n)
        slot = int(state_indices[b])
        hist = _f32(conv_state[slot]) if bool(has_state[b]) else torch.zeros_like(conv_state[slot], dtype=torch.float32)
        seq = torch.cat([hist, _f32(x[off:off + n]).t()], dim=1)          # [C, K-1+n]
        y = F.conv1d(seq.unsqueeze(0), _f32(weight).unsqueeze(1), None, groups=weight.shape[0]).squeeze(0)  # [C, n]
        out[off:off + n] = F.silu(y).t().to(x.dtype)
        conv_state[slot] = seq[:, -(K - 1):].to(conv_state.dtype)
        off += n
    return out


def gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                     state: torch.Tensor, state_indices: torch.Tensor, seq_lens, has_state) -> torch.Tensor:
    """Recurrent gated delta rule, one token at a time (the definition the chunked forms must match).

    q, k [T, H, Dk] (l2-normalised here, q scaled by Dk^-0.5), v [T, H, Dv], g (log decay) and beta [T, H];
    ``state`` [slots, H, Dk, Dv] fp32 is read when ``has_state[b]`` and always written back:
    ``S *= exp(g); S += k (x) ((v - S^T k) * beta); o = S^T q``."""
    T, H, Dk = q.shape
    qf = _f32(q)
    kf = _f32(k)
    qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * Dk ** -0.5
    kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    vf, gf, bf = _f32(v), _f32(g), _f32(beta)
    out = torch.empty(T, H, v.shape[-1], dtype=torch.float32, device=q.device)
    off = 0
    for b, n in enumerate(list(seq_lens)):
        n = int(n)
        slot = int(state_indices[b])
        S = state[slot].float().clone() if bool(has_state[b]) else torch.zeros_like(state[slot], dtype=torch.float32)
        for t in range(off, off + n):
            S = S * gf[t].exp().view(H, 1, 1)
            mem = (S * kf[t].unsqueeze(-1)).sum(-2)                        # [H, Dv]
            delta = (vf[t] - mem) * bf[t].unsqueeze(-1)
            S = S + kf[t].unsqueeze(-1) * delta.unsqueeze(-2)
            out[t] = (S * qf[t].unsqueeze(-1)).sum(-2)
        state[slot] = S.to(state.dtype)
        off += n
    return out.to(v.dtype)



def gated_delta_rule_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                             state: torch.Tensor, state_indices: torch.Tensor, seq_lens, has_state,
                             chunk: int = 64) -> torch.Tensor:
    """The same rule as :func:`gated_delta_rule`, evaluated ``chunk`` tokens at a time with matrix
    products (the chunk-parallel form used for prefill; role of pymllm's ``gdn_chunkwise`` reference).

    Inside a chunk with cumulative log decay ``G_i = sum_{j<=i} g_j`` and incoming state ``S0``:

        A[i, j] = exp(G_i - G_j) (k_i . k_j)  for j < i          (strictly lower triangular)
        U       = (I + diag(beta) A)^-1 diag(beta) (V - exp(G) * (K S0))      # the per-token updates
        O       = exp(G) * (Q S0) + (M * (Q K^T)) U,   M[i, j] = exp(G_i - G_j) for j <= i
        S_end   = exp(G_C) S0 + (exp(G_C - G) * K)^T U

    All exponents are of non-positive numbers (``g <= 0``), so nothing overflows."""
    T, H, Dk = q.shape
    qf = _f32(q)
    kf = _f32(k)
    qf = qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * Dk ** -0.5
    kf = kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
    vf, gf, bf = _f32(v), _f32(g), _f32(beta)
    out = torch.empty(T, H, v.shape[-1], dtype=torch.float32, device=q.device)
    off = 0
    for b, n in enumerate(list(seq_lens)):
        n = int(n)
        slot = int(state_indices[b])
        S = state[slot].float().clone() if bool(has_state[b]) else torch.zeros_like(state[slot], dtype=torch.float32)
        for c0 in range(off, off + n, chunk):
            c1 = min(off + n, c0 + chunk)
            C = c1 - c0
            Q, K, V = (t[c0:c1].transpose(0, 1) for t in (qf, kf, vf))          # [H, C, D]
            G = gf[c0:c1].transpose(0, 1).cumsum(-1)                            # [H, C]
            B = bf[c0:c1].transpose(0, 1)                                       # [H, C]
            diff = G.unsqueeze(-1) - G.unsqueeze(-2)                            # G_i - G_j
            lower = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
            M = torch.where(lower, diff, torch.full_like(diff, float("-inf"))).exp()   # j <= i
            A = (M * (K @ K.transpose(-1, -2))).tril(-1)
            eG = G.exp().unsqueeze(-1)
            rhs = B.unsqueeze(-1) * (V - eG * (K @ S))
            lhs = torch.eye(C, device=q.device, dtype=torch.float32) + B.unsqueeze(-1) * A
            U = torch.linalg.solve_triangular(lhs, rhs, upper=False, unitriangular=True)
            out[c0:c1] = (eG * (Q @ S) + (M * (Q @ K.transpose(-1, -2))) @ U).transpose(0, 1)
            tail = (G[:, -1:] - G).exp().unsqueeze(-1)                          # exp(G_C - G_j)
            S = G[:, -1].exp().view(H, 1, 1) * S + (tail * K).transpose(-1, -2) @ U
        state[slot] = S.to(state.dtype)
        off += n
    return out.to(v.dtype)

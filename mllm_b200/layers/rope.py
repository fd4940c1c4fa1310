"""Stand-alone rotary-embedding operators under the reference's names (pymllm/layers/rope.py:16-640).

The serving path does not call these: RoPE / M-RoPE is fused with the per-head QK-norm and the KV-cache
write in one kernel (`ops.qk_norm_rope_kv_write`).  They exist for API parity (ragged ``indptr`` +
``offsets`` form, explicit position ids, llama-3.1 frequency scaling, cos/sin-cache form, M-RoPE) and
compute in fp32 with one rounding to the input type.
"""

from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch


def _positions_from_ragged(indptr: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    lens = (indptr[1:] - indptr[:-1]).long()
    seg = torch.repeat_interleave(torch.arange(lens.numel(), device=indptr.device), lens)
    within = torch.arange(int(lens.sum()), device=indptr.device) - indptr[:-1].long()[seg]
    return within + offsets.long()[seg]


def _inv_freq(rotary_dim: int, theta: float, device, llama31: Optional[Tuple[float, float, float, float]] = None) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, device=device, dtype=torch.float32) / rotary_dim))
    if llama31 is not None:
        scale, low, high, old_len = llama31
        wavelen = 2 * math.pi / inv
        smooth = ((old_len / wavelen - low) / (high - low)).clamp(0, 1)
        inv = (1 - smooth) * inv / scale + smooth * inv
    return inv


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleave: bool) -> torch.Tensor:
    """x [T, H, D]; cos/sin [T, rd/2]; rotates the first rd features."""
    rd = cos.shape[-1] * 2
    xf = x.float()
    rot, rest = xf[..., :rd], xf[..., rd:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    if interleave:
        a, b = rot[..., 0::2], rot[..., 1::2]
        out = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    else:
        a, b = rot[..., : rd // 2], rot[..., rd // 2:]
        out = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    return torch.cat([out, rest], dim=-1).to(x.dtype)


def _apply(q, k, pos, rotary_dim, interleave, rope_scale, rope_theta, inplace, llama31=None):
    rd = rotary_dim or q.shape[-1]
    ang = (pos.float() / rope_scale).unsqueeze(-1) * _inv_freq(rd, rope_theta, q.device, llama31)
    qo, ko = _rotate(q, ang.cos(), ang.sin(), interleave), _rotate(k, ang.cos(), ang.sin(), interleave)
    if inplace:
        q.copy_(qo)
        k.copy_(ko)
        return None
    return qo, ko


def apply_rope(q, k, indptr, offsets, inplace: bool = False, rotary_dim: Optional[int] = None, interleave: bool = False,
               rope_scale: float = 1.0, rope_theta: float = 1e4):
    return _apply(q, k, _positions_from_ragged(indptr, offsets), rotary_dim, interleave, rope_scale, rope_theta, inplace)


def apply_rope_pos_ids(q, k, pos_ids, inplace: bool = False, rotary_dim: Optional[int] = None, interleave: bool = False,
                       rope_scale: float = 1.0, rope_theta: float = 1e4):
    return _apply(q, k, pos_ids, rotary_dim, interleave, rope_scale, rope_theta, inplace)


def apply_llama31_rope(q, k, indptr, offsets, inplace: bool = False, rotary_dim: Optional[int] = None, interleave: bool = False,
                       rope_scale: float = 8.0, rope_theta: float = 5e5, low_freq_factor: float = 1.0,
                       high_freq_factor: float = 4.0, old_context_len: int = 8192):
    return _apply(q, k, _positions_from_ragged(indptr, offsets), rotary_dim, interleave, 1.0, rope_theta, inplace,
                  (rope_scale, low_freq_factor, high_freq_factor, float(old_context_len)))


def apply_llama31_rope_pos_ids(q, k, pos_ids, inplace: bool = False, rotary_dim: Optional[int] = None, interleave: bool = False,
                               rope_scale: float = 8.0, rope_theta: float = 5e5, low_freq_factor: float = 1.0,
                               high_freq_factor: float = 4.0, old_context_len: int = 8192):
    return _apply(q, k, pos_ids, rotary_dim, interleave, 1.0, rope_theta, inplace,
                  (rope_scale, low_freq_factor, high_freq_factor, float(old_context_len)))


def apply_rope_with_cos_sin_cache(positions, query, key, head_size: int, cos_sin_cache, inplace: bool = False,
                                  is_neox: bool = True):
    """``query`` / ``key`` are ``[T, heads * head_size]``; the cache row holds ``[cos(rd/2) | sin(rd/2)]``."""
    cs = cos_sin_cache[positions.long()].float()
    half = cs.shape[-1] // 2
    cos, sin = cs[..., :half], cs[..., half:]
    q3, k3 = query.view(query.shape[0], -1, head_size), key.view(key.shape[0], -1, head_size)
    qo = _rotate(q3, cos, sin, not is_neox).view_as(query)
    ko = _rotate(k3, cos, sin, not is_neox).view_as(key)
    if inplace:
        query.copy_(qo)
        key.copy_(ko)
        return None
    return qo, ko


def apply_mrope(q, k, positions, cos_sin_cache, mrope_section: List[int], mrope_interleaved: bool = True):
    """M-RoPE: ``positions`` [3, T] (t, h, w); frequency i takes its angle from the axis chosen by
    ``mrope_section`` (consecutive sections, or interleaved t/h/w).  q, k: ``[T, H, D]``."""
    half = cos_sin_cache.shape[-1] // 2
    cs = cos_sin_cache[positions.long()].float()              # [3, T, 2*half]
    axis = _mrope_axis(half, mrope_section, mrope_interleaved, q.device)
    idx = axis.view(1, 1, half).expand(1, cs.shape[1], half)
    cos = cs[..., :half].gather(0, idx).squeeze(0)
    sin = cs[..., half:].gather(0, idx).squeeze(0)
    return _rotate(q, cos, sin, False), _rotate(k, cos, sin, False)


def apply_mrope_fused_(q, k, positions, cos_sin_cache, mrope_section: List[int], mrope_interleaved: bool = True) -> None:
    """In-place form of :func:`apply_mrope`."""
    qo, ko = apply_mrope(q, k, positions, cos_sin_cache, mrope_section, mrope_interleaved)
    q.copy_(qo)
    k.copy_(ko)


def _mrope_axis(half: int, sections: List[int], interleaved: bool, device) -> torch.Tensor:
    axis = torch.zeros(half, dtype=torch.long, device=device)
    if interleaved:
        for a in (1, 2):
            n = sections[a] * 3
            axis[torch.arange(a, min(n, half), 3, device=device)] = a
    else:
        s0, s1 = sections[0], sections[0] + sections[1]
        axis[s0:s1] = 1
        axis[s1: s1 + sections[2]] = 2
    return axis

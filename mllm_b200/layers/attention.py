"""Model-side attention layer over the slot-indexed KV pool.

Holds head counts, scale and the layer index (as pymllm/layers/attention/radix_attention.py:24-171)
and runs the fused prologue (per-head QK-norm, rotary embedding, cache write) followed by
the prefill or decode attention kernel chosen by the batch's forward mode.  The kernels read
the request->slot table directly, so there is no per-step planning or index flattening.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops


class RadixAttention(nn.Module):
    def __init__(self, num_heads: int, head_dim: int, scaling: float, num_kv_heads: int, layer_id: int,
                 rope_theta: float = 1e6, rms_eps: float = 1e-6, mrope_sections=None,
                 mrope_interleaved: bool = False, rope_scaling: Optional[dict] = None,
                 sliding_window: Optional[int] = None, logit_cap: float = 0.0) -> None:
        super().__init__()
        self.rope_scaling = rope_scaling
        # each query attends to its last `sliding_window` keys (itself included); scores soft-capped at logit_cap
        self.sliding_window = int(sliding_window) if sliding_window else None
        self.logit_cap = float(logit_cap or 0.0)
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        # yarn / longrope checkpoints scale cos and sin by a constant: q.k grows by its square
        self.scaling, self.layer_id = scaling * ops.rope_attention_factor(rope_scaling) ** 2, layer_id
        self.rope_theta, self.rms_eps = rope_theta, rms_eps
        self.mrope_sections, self.mrope_interleaved = mrope_sections, mrope_interleaved
        self._inv_freq: Optional[torch.Tensor] = None
        self._axis_map: Optional[torch.Tensor] = None

    def _tables(self, device):
        if self._inv_freq is None or self._inv_freq.device != device:
            self._inv_freq = ops.rope_inv_freq(self.head_dim, self.rope_theta, device, self.rope_scaling)
            if self.mrope_sections is not None:
                self._axis_map = ops.mrope_axis_map(self.head_dim, self.mrope_sections, self.mrope_interleaved, device)
        return self._inv_freq, self._axis_map

    def forward(self, qkv: torch.Tensor, q_norm_w, k_norm_w, forward_batch) -> torch.Tensor:
        """``qkv`` [T, (Hq+2Hkv)*D] fused projection output -> attention output [T, Hq*D]."""
        fb = forward_batch
        T = qkv.shape[0]
        if fb.forward_mode.is_idle() or T == 0:
            return qkv.new_zeros((T, self.num_heads * self.head_dim))
        k_cache, v_cache = fb.token_to_kv_pool.get_kv_buffer(self.layer_id)
        inv_freq, axis_map = self._tables(qkv.device)
        use_mrope = self.mrope_sections is not None and fb.mrope_positions is not None
        ops.qk_norm_rope_kv_write(
            qkv, q_norm_w, k_norm_w, fb.mrope_positions if use_mrope else fb.positions, fb.out_cache_loc,
            k_cache, v_cache, self.num_heads, self.num_kv_heads, self.head_dim, self.rope_theta, self.rms_eps,
            self.mrope_sections if use_mrope else None, self.mrope_interleaved,
            inv_freq=inv_freq, axis_map=axis_map if use_mrope else None,
        )
        q = qkv[:, : self.num_heads * self.head_dim].view(T, self.num_heads, self.head_dim)
        out = torch.empty((T, self.num_heads, self.head_dim), dtype=qkv.dtype, device=qkv.device)
        if fb.forward_mode.is_decode():
            ops.attention_decode(q, k_cache, v_cache, fb.req_to_token_pool.req_to_token, fb.req_pool_indices,
                                 fb.seq_lens, self.scaling, out=out, max_seq_len=fb.max_seq_len,
                                 window=self.sliding_window, logit_cap=self.logit_cap)
        else:
            ops.attention_prefill(q, k_cache, v_cache, fb.req_to_token_pool.req_to_token, fb.req_pool_indices,
                                  fb.seq_lens, fb.extend_prefix_lens, fb.extend_start_loc, self.scaling, out=out,
                                  max_q_len=fb.max_extend_len, window=self.sliding_window, logit_cap=self.logit_cap)
        return out.view(T, self.num_heads * self.head_dim)

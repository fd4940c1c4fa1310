"""Qwen2.5-VL (``Qwen2_5_VLForConditionalGeneration``; ``mllm/models/qwen2_5vl`` in the reference's C++ runtime): Qwen2 decoder with sectioned 3-D rope, behind a
vision tower with RMSNorm blocks, SwiGLU MLPs and *windowed* attention: patches are reordered (in units of
one merged 2 x 2 token) so that every ``window_size`` square is contiguous, most blocks attend inside a
window, the blocks listed in ``fullatt_block_indexes`` attend over the whole image, and the merged tokens
are put back in raster order at the end.  Attention, GEMMs and the merger run on the same kernels as the
Qwen3-VL tower; only the segment boundaries handed to the variable-length attention differ per block."""

from __future__ import annotations

from types import SimpleNamespace
from typing import Iterable, List, Optional, Tuple

import numpy as np
import torch
from torch import nn

from .. import ops
from ..layers import RMSNorm
from .llama import Qwen2ForCausalLM
from .qwen3_vl import VisionAttention, VisionLanguageMixin, _Linear, rot_pos_ids


class _SwiGLUMLP(nn.Module):
    def __init__(self, dim: int, inter: int, dtype) -> None:
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = _Linear(dim, inter, dtype), _Linear(dim, inter, dtype), _Linear(inter, dim, dtype)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class _Block(nn.Module):
    def __init__(self, dim: int, heads: int, inter: int, dtype) -> None:
        super().__init__()
        self.norm1, self.norm2 = RMSNorm(dim, 1e-6, dtype), RMSNorm(dim, 1e-6, dtype)
        self.attn = VisionAttention(dim, heads, dtype)
        self.mlp = _SwiGLUMLP(dim, inter, dtype)

    def forward(self, x, cu, cos, sin):
        x = x + self.attn(self.norm1(x), cu, cos, sin)
        return x + self.mlp(self.norm2(x))


class _Merger(nn.Module):
    def __init__(self, out_dim: int, context_dim: int, merge: int, dtype) -> None:
        super().__init__()
        self.hidden = context_dim * merge * merge
        self.ln_q = RMSNorm(context_dim, 1e-6, dtype)
        self.mlp = nn.ModuleList([_Linear(self.hidden, self.hidden, dtype), nn.Identity(), _Linear(self.hidden, out_dim, dtype)])

    def forward(self, x):
        return self.mlp[2](ops.gelu_erf(self.mlp[0](self.ln_q(x).reshape(-1, self.hidden))))


def window_order(grids: List[List[int]], window: int, merge: int, patch: int):
    """(order of the merged tokens that makes every attention window contiguous, window boundaries in
    patches).  Windows are ``window / merge / patch`` merged tokens on a side; edge windows are smaller."""
    side = window // merge // patch
    unit = merge * merge
    order, cu, base = [], [0], 0
    for t, h, w in grids:
        gh, gw = h // merge, w // merge
        idx = np.arange(t * gh * gw).reshape(t, gh, gw)
        ph, pw = side - gh % side, side - gw % side          # a full extra window when already aligned, as the model does
        pad = np.full((t, gh + ph, gw + pw), -1, dtype=np.int64)
        pad[:, :gh, :gw] = idx
        nh, nw = (gh + ph) // side, (gw + pw) // side
        win = pad.reshape(t, nh, side, nw, side).transpose(0, 1, 3, 2, 4).reshape(t * nh * nw, side * side)
        for row in win:
            keep = row[row >= 0]
            if keep.size:
                order.append(keep + base)
                cu.append(cu[-1] + int(keep.size) * unit)
        base += t * gh * gw
    return np.concatenate(order), np.asarray(cu, dtype=np.int32)


class Qwen2_5VisionModel(nn.Module):
    def __init__(self, vc, dtype) -> None:
        super().__init__()
        self.hidden_size, self.num_heads = vc.hidden_size, vc.num_heads
        self.patch_size, self.temporal_patch_size = vc.patch_size, getattr(vc, "temporal_patch_size", 2)
        self.spatial_merge_size = getattr(vc, "spatial_merge_size", 2)
        self.window_size = getattr(vc, "window_size", 112)
        self.fullatt_block_indexes = list(getattr(vc, "fullatt_block_indexes", [7, 15, 23, 31]))
        self.deepstack_visual_indexes: List[int] = []
        patch_dim = getattr(vc, "in_channels", 3) * self.temporal_patch_size * self.patch_size * self.patch_size
        self.patch_embed = nn.Module()
        self.patch_embed.proj = _Linear(patch_dim, vc.hidden_size, dtype)
        self.blocks = nn.ModuleList(_Block(vc.hidden_size, vc.num_heads, vc.intermediate_size, dtype) for _ in range(vc.depth))
        self.merger = _Merger(vc.out_hidden_size, vc.hidden_size, self.spatial_merge_size, dtype)
        rotary_dim = vc.hidden_size // vc.num_heads // 2
        self._inv_freq = torch.from_numpy(1.0 / (10000.0 ** (np.arange(0, rotary_dim, 2, dtype=np.float32) / rotary_dim)))

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        grids = grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else [list(g) for g in grid_thw]
        w = self.patch_embed.proj.weight
        x = self.patch_embed.proj(pixel_values.to(device=w.device, dtype=w.dtype).reshape(pixel_values.shape[0], -1))
        unit = self.spatial_merge_size ** 2
        order, cu_win = window_order(grids, self.window_size, self.spatial_merge_size, self.patch_size)
        order_t = torch.from_numpy(order).to(w.device)
        pos = torch.cat([rot_pos_ids(h, wd, self.spatial_merge_size).repeat(t, 1) for t, h, wd in grids], 0).float()
        freqs = (pos.unsqueeze(-1) * self._inv_freq).flatten(1).to(w.device)            # [T, head_dim / 2], raster-merge order
        x = x.reshape(-1, unit, x.shape[-1])[order_t].reshape(-1, x.shape[-1])
        freqs = freqs.reshape(-1, unit, freqs.shape[-1])[order_t].reshape(-1, freqs.shape[-1])
        cos, sin = freqs.cos(), freqs.sin()
        lens = np.repeat([g[1] * g[2] for g in grids], [g[0] for g in grids])
        cu_full = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32))
        cu_win_t = torch.from_numpy(cu_win)
        for i, blk in enumerate(self.blocks):
            x = blk(x, cu_full if i in self.fullatt_block_indexes else cu_win_t, cos, sin)
        merged = self.merger(x)
        return merged[torch.from_numpy(np.argsort(order)).to(w.device)]


class Qwen2_5_VLForConditionalGeneration(VisionLanguageMixin, Qwen2ForCausalLM):
    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None) -> None:
        tc = getattr(config, "text_config", config)
        rs = getattr(tc, "rope_scaling", None) or getattr(tc, "rope_parameters", None) or {}
        rs = rs if isinstance(rs, dict) else vars(rs)
        if not hasattr(tc, "tie_word_embeddings"):
            tc.tie_word_embeddings = bool(getattr(config, "tie_word_embeddings", False))
        Qwen2ForCausalLM.__init__(self, tc, quant_config, params_dtype, mrope_sections=rs.get("mrope_section", [16, 24, 24]),
                                  mrope_interleaved=False)
        dt = params_dtype or torch.get_default_dtype()
        self.full_config = config
        self.visual = Qwen2_5VisionModel(config.vision_config, dt)
        self.image_token_id = config.image_token_id
        self.video_token_id = getattr(config, "video_token_id", None)
        self.vision_start_token_id = config.vision_start_token_id
        self.spatial_merge_size = self.visual.spatial_merge_size
        self.num_deepstack = 0
        self.hidden_size = tc.hidden_size

    def forward(self, input_ids, positions, forward_batch, input_embeds=None):
        fb = forward_batch
        self._set_mrope_positions(input_ids, fb)
        embeds, _ = self._vision_embeds(input_ids, fb)
        return Qwen2ForCausalLM.forward(self, input_ids, positions, fb, embeds if embeds is not None else input_embeds)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        loaded, rest = self._load_visual(weights)
        return loaded | Qwen2ForCausalLM.load_weights(self, rest)


EntryClass = Qwen2_5_VLForConditionalGeneration

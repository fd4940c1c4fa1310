"""Qwen3-VL (Qwen3VLForConditionalGeneration): vision tower + Qwen3 decoder with interleaved M-RoPE
and deepstack injection.

Semantics follow pymllm/models/qwen3_vl.py: Conv3d patch embedding as one GEMM over flattened
``[N, C*T*P*P]`` patches (:78-115), bilinearly interpolated learned position embedding (:402-491),
2-D rotary embedding (:343-400), ``depth`` pre-LayerNorm blocks with bidirectional per-image attention
and a GELU-tanh MLP (:125-221), a 2x2 patch merger plus one post-shuffle-norm merger per deepstack index
(:224-255, :495-548), image-token scatter and per-token deepstack tensors (:1246-1272), 3-D position ids
(:595-694) and the per-request position delta used by decode (:1196-1210).

Here the whole tower runs on the sm_100a kernels: every projection is a tcgen05 GEMM with the bias in
its epilogue, attention is the tcgen05 prefill kernel without causal mask (one launch for all images
instead of a per-image loop with host syncs), RoPE + q/k/v split + head padding is one kernel, and the
position-embedding interpolation is one gather-add kernel.  The tower is replicated on every
tensor-parallel rank (it is small next to the decoder); the decoder is the tensor-parallel Qwen3.
"""

from __future__ import annotations

import os

import time
from typing import Iterable, List, Optional, Tuple

import numpy as np
import torch
from torch import nn

from .. import ops
from ..engine.forward_batch import ForwardBatch
from ..layers import LayerNorm
from .qwen3 import LogitsProcessorOutput, Qwen3ForCausalLM


def _text_config(config):
    return getattr(config, "text_config", config)


class _Linear(nn.Module):
    """Replicated linear layer with bias on the tcgen05 GEMM."""

    def __init__(self, in_features: int, out_features: int, dtype) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)


class VisionAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, dtype) -> None:
        super().__init__()
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.qkv = _Linear(dim, 3 * dim, dtype)
        self.proj = _Linear(dim, dim, dtype)

    def forward(self, x, cu_seqlens, cos, sin):
        o = ops.vision_attention(self.qkv(x), cos, sin, cu_seqlens, self.num_heads, self.head_dim ** -0.5)
        return self.proj(o)


class VisionMLP(nn.Module):
    def __init__(self, dim: int, inter: int, act: str, dtype) -> None:
        super().__init__()
        self.linear_fc1 = _Linear(dim, inter, dtype)
        self.linear_fc2 = _Linear(inter, dim, dtype)
        acts = {"gelu_pytorch_tanh": ops.gelu_tanh, "gelu": ops.gelu_erf,
                "quick_gelu": lambda x: x * torch.sigmoid(1.702 * x)}
        if act not in acts:
            raise ValueError(f"unsupported vision activation {act!r}")
        self.act = acts[act]

    def forward(self, x):
        return self.linear_fc2(self.act(self.linear_fc1(x)))


class VisionBlock(nn.Module):
    def __init__(self, dim: int, num_heads: int, inter: int, act: str, eps: float, dtype) -> None:
        super().__init__()
        self.norm1 = LayerNorm(dim, eps, params_dtype=dtype)
        self.norm2 = LayerNorm(dim, eps, params_dtype=dtype)
        self.attn = VisionAttention(dim, num_heads, dtype)
        self.mlp = VisionMLP(dim, inter, act, dtype)

    def forward(self, x, cu_seqlens, cos, sin):
        x = x + self.attn(self.norm1(x), cu_seqlens, cos, sin)
        return x + self.mlp(self.norm2(x))


class PatchMerger(nn.Module):
    """Groups ``merge**2`` consecutive tokens; LayerNorm before (main merger) or after (deepstack
    mergers) the grouping, then fc1 -> exact GELU -> fc2."""

    def __init__(self, out_dim: int, context_dim: int, merge: int, post_shuffle_norm: bool, eps: float, dtype) -> None:
        super().__init__()
        self.hidden = context_dim * merge * merge
        self.post_shuffle_norm = post_shuffle_norm
        self.norm = LayerNorm(self.hidden if post_shuffle_norm else context_dim, eps, params_dtype=dtype)
        self.linear_fc1 = _Linear(self.hidden, self.hidden, dtype)
        self.linear_fc2 = _Linear(self.hidden, out_dim, dtype)

    def forward(self, x):
        x = self.norm(x.reshape(-1, self.hidden)) if self.post_shuffle_norm else self.norm(x).reshape(-1, self.hidden)
        return self.linear_fc2(ops.gelu_erf(self.linear_fc1(x)))


def rot_pos_ids(h: int, w: int, merge: int) -> torch.Tensor:
    """(row, column) of every patch in merger order: ``merge x merge`` neighbours are consecutive."""
    hi = torch.arange(h).unsqueeze(1).expand(-1, w).reshape(h // merge, merge, w // merge, merge)
    wi = torch.arange(w).unsqueeze(0).expand(h, -1).reshape(h // merge, merge, w // merge, merge)
    return torch.stack([hi.permute(0, 2, 1, 3).flatten(), wi.permute(0, 2, 1, 3).flatten()], dim=-1)


def interpolation_indices_and_weights(h: int, w: int, side: int):
    """Bilinear corners of an ``h x w`` grid sampled from the learned ``side x side`` table:
    four index arrays and four weight arrays of length ``h * w`` (row-major)."""
    hi = np.linspace(0, side - 1, h, dtype=np.float32)
    wi = np.linspace(0, side - 1, w, dtype=np.float32)
    hf, wf = np.floor(hi).astype(np.int64), np.floor(wi).astype(np.int64)
    hc, wc = np.clip(hf + 1, 0, side - 1), np.clip(wf + 1, 0, side - 1)
    dh, dw = hi - hf, wi - wf
    idx = [(hf[:, None] * side + wf).flatten(), (hf[:, None] * side + wc).flatten(),
           (hc[:, None] * side + wf).flatten(), (hc[:, None] * side + wc).flatten()]
    wts = [((1 - dh)[:, None] * (1 - dw)).flatten(), ((1 - dh)[:, None] * dw).flatten(),
           (dh[:, None] * (1 - dw)).flatten(), (dh[:, None] * dw).flatten()]
    return idx, wts


class Qwen3VLVisionModel(nn.Module):
    def __init__(self, vc, dtype) -> None:
        super().__init__()
        self.hidden_size = vc.hidden_size
        self.num_heads = vc.num_heads
        self.patch_size, self.temporal_patch_size = vc.patch_size, getattr(vc, "temporal_patch_size", 2)
        self.spatial_merge_size = getattr(vc, "spatial_merge_size", 2)
        self.in_channels = getattr(vc, "in_channels", 3)
        self.deepstack_visual_indexes = list(getattr(vc, "deepstack_visual_indexes", None) or [])
        # towers without a learned position table (Qwen2-VL) rely on the 2-D rotary embedding alone
        self.num_position_embeddings = int(getattr(vc, "num_position_embeddings", 0) or 0)
        self.side = int(self.num_position_embeddings ** 0.5)
        eps = getattr(vc, "norm_eps", 1e-6)
        patch_dim = self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size
        self.patch_embed = nn.Module()
        self.patch_embed.proj = _Linear(patch_dim, vc.hidden_size, dtype)  # Conv3d with kernel == stride
        if self.num_position_embeddings:
            self.pos_embed = nn.Module()
            self.pos_embed.weight = nn.Parameter(torch.empty(self.num_position_embeddings, vc.hidden_size, dtype=dtype),
                                                 requires_grad=False)
        self.blocks = nn.ModuleList(
            VisionBlock(vc.hidden_size, vc.num_heads, vc.intermediate_size, getattr(vc, "hidden_act", "gelu_pytorch_tanh"),
                        eps, dtype) for _ in range(vc.depth))
        self.merger = PatchMerger(vc.out_hidden_size, vc.hidden_size, self.spatial_merge_size, False, eps, dtype)
        self.deepstack_merger_list = nn.ModuleList(
            PatchMerger(vc.out_hidden_size, vc.hidden_size, self.spatial_merge_size, True, eps, dtype)
            for _ in self.deepstack_visual_indexes)
        head_dim = vc.hidden_size // vc.num_heads
        rotary_dim = head_dim // 2
        # host-side table (the module may be constructed under a device context)
        self._inv_freq = torch.from_numpy(1.0 / (10000.0 ** (np.arange(0, rotary_dim, 2, dtype=np.float32) / rotary_dim)))

    # -- host-side index building (cheap; depends only on the grids) --
    def rotary_cos_sin(self, grids: List[List[int]], device) -> Tuple[torch.Tensor, torch.Tensor]:
        ids = []
        for t, h, w in grids:
            base = rot_pos_ids(h, w, self.spatial_merge_size)
            ids.append(base if t == 1 else base.repeat(t, 1))
        pos = torch.cat(ids, 0).float()                                   # [T, 2]
        freqs = pos.unsqueeze(-1) * self._inv_freq                         # [T, 2, rotary_dim / 2]
        freqs = freqs.flatten(1).to(device)                                # [T, head_dim / 2]
        return freqs.cos(), freqs.sin()

    def pos_embed_indices(self, grids: List[List[int]], device):
        merge = self.spatial_merge_size
        idx_parts, w_parts = [], []
        for t, h, w in grids:
            idx, wts = interpolation_indices_and_weights(h, w, self.side)
            # reorder row-major patches into merger order, repeat over the temporal extent
            order = torch.arange(h * w).view(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten().numpy()
            idx_parts.append(np.tile(np.stack(idx)[:, order], (1, t)))
            w_parts.append(np.tile(np.stack(wts)[:, order], (1, t)))
        idx = torch.from_numpy(np.concatenate(idx_parts, 1)).to(device)
        wts = torch.from_numpy(np.concatenate(w_parts, 1).astype(np.float32)).to(device)
        return idx, wts

    def _tables(self, grids: List[List[int]], rows: int, device):
        """Everything that depends on the grids only: position-table indices and weights, rotary tables, and the
        attention plan (segment boundaries on the device, row table).  Built on the host once per call."""
        idx = wts = None
        if self.num_position_embeddings:
            idx, wts = self.pos_embed_indices(grids, device)
        cos, sin = self.rotary_cos_sin(grids, device)
        lens = np.repeat([g[1] * g[2] for g in grids], [g[0] for g in grids])
        cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32))
        return idx, wts, cos.float().contiguous(), sin.float().contiguous(), ops.VarlenPlan(cu, rows, device)

    def _tower(self, pixels: torch.Tensor, tables) -> torch.Tensor:
        """The device part: patch projection, position table, blocks, mergers.  No host work, no synchronisation:
        this is what a CUDA graph holds."""
        idx, wts, cos, sin, plan = tables
        x = self.patch_embed.proj(pixels)
        if idx is not None:
            x = ops.vision_pos_embed_add(x, self.pos_embed.weight, idx, wts)
        feats = []
        ds = 0
        for i, blk in enumerate(self.blocks):
            x = blk(x, plan, cos, sin)
            if i in self.deepstack_visual_indexes:
                feats.append(self.deepstack_merger_list[ds](x))
                ds += 1
        return torch.cat([self.merger(x)] + feats, dim=-1)

    # Captured towers, keyed by the grids of a call.  The tower is a few hundred small launches (≈7.5 ms for one
    # 448 x 448 image when issued one by one); a graph replays them in a fraction of that.  Kept small: every
    # graph owns its activations.
    _GRAPH_CACHE_ENTRIES = 8
    _GRAPH_MAX_PATCHES = 16384

    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        """``pixel_values`` [total_patches, C*T*P*P]; returns ``[merged_tokens, out_hidden * (1 + deepstack)]``."""
        grids = grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else [list(g) for g in grid_thw]
        w = self.patch_embed.proj.weight
        pixels = pixel_values.to(device=w.device, dtype=w.dtype).reshape(pixel_values.shape[0], -1)
        use_graph = (w.is_cuda and os.environ.get("MLLM_B200_VIT_GRAPH", "1") != "0" and ops.use_kernels(pixels)
                     and pixels.shape[0] <= self._GRAPH_MAX_PATCHES and not torch.cuda.is_current_stream_capturing())
        if not use_graph:
            return self._tower(pixels, self._tables(grids, pixels.shape[0], w.device))
        cache = self.__dict__.setdefault("_graphs", {})
        key = (tuple(tuple(int(v) for v in g) for g in grids), tuple(pixels.shape), pixels.dtype)
        entry = cache.pop(key, None)
        if entry is None:
            tables = self._tables(grids, pixels.shape[0], w.device)
            static_in = pixels.clone()
            stream = torch.cuda.Stream(device=w.device)
            stream.wait_stream(torch.cuda.current_stream(w.device))
            with torch.cuda.stream(stream):
                self._tower(static_in, tables)            # first run outside the capture: lazy initialisation, allocator warm-up
            torch.cuda.current_stream(w.device).wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                static_out = self._tower(static_in, tables)
            entry = (graph, static_in, static_out, tables)
            while len(cache) >= self._GRAPH_CACHE_ENTRIES:
                cache.pop(next(iter(cache)))
        cache[key] = entry                                # most recently used last
        graph, static_in, static_out, _ = entry
        static_in.copy_(pixels)
        graph.replay()
        return static_out.clone()


def get_rope_index(input_ids: torch.Tensor, image_grid_thw, image_token_id: int, vision_start_token_id: int,
                   spatial_merge_size: int, start: int = 0, t_scales=None) -> Tuple[torch.Tensor, int]:
    """3-D (t, h, w) position ids of one sequence and ``delta = next_position - len``.

    Text tokens advance all three axes together; the tokens of an image that follows a vision-start
    token take ``base + (t, h, w)`` of the merged grid and the counter then jumps to one past the
    largest position used (``max(t, h, w)`` when time is not scaled).  ``start`` is the first position
    (a cached prefix of text).  ``t_scales`` holds one factor per grid for the temporal axis: a video clip
    of Qwen2.5-VL advances ``seconds per temporal patch x tokens per second`` positions per temporal patch
    (truncated to an integer per patch); 1 everywhere else."""
    ids = input_ids.tolist()
    T = len(ids)
    grids = [] if image_grid_thw is None else (image_grid_thw.tolist() if isinstance(image_grid_thw, torch.Tensor)
                                               else [list(g) for g in image_grid_thw])
    pos = np.zeros((3, T), dtype=np.int64)
    cur, img, i = start, 0, 0
    while i < T:
        if ids[i] == vision_start_token_id and img < len(grids):
            pos[:, i] = cur
            cur += 1
            i += 1
            t, h, w = int(grids[img][0]), int(grids[img][1]) // spatial_merge_size, int(grids[img][2]) // spatial_merge_size
            n = min(t * h * w, T - i)
            steps = np.arange(t)
            if t_scales is not None and float(t_scales[img]) != 1.0:
                steps = (steps * float(t_scales[img])).astype(np.int64)
            tt, hh, ww = np.meshgrid(steps, np.arange(h), np.arange(w), indexing="ij")
            pos[0, i:i + n] = tt.flatten()[:n] + cur
            pos[1, i:i + n] = hh.flatten()[:n] + cur
            pos[2, i:i + n] = ww.flatten()[:n] + cur
            cur += max(int(steps[-1]) + 1, h, w)
            i += n
            img += 1
        else:
            pos[:, i] = cur
            cur += 1
            i += 1
    return torch.from_numpy(pos).to(input_ids.device), cur - start - T


class VisionLanguageMixin:
    """What the vision-language variants share on top of their text model: 3-D rope positions of a
    prompt with image blocks, and image features written over the image-token rows of the input
    embeddings.  The host class provides ``visual``, ``image_token_id``, ``vision_start_token_id``,
    ``spatial_merge_size``, ``hidden_size``, ``num_deepstack`` and ``model.embed_tokens``."""

    uses_mrope = True
    # videos: rows that carry this token take features like image rows.  Qwen3-VL prompts hold one block per
    # temporal patch (grid [1, h, w] each); Qwen2-VL / Qwen2.5-VL prompts hold one block per clip (grid [T, h, w])
    video_token_id: Optional[int] = None

    def _init_vision(self, config, dtype) -> None:
        self.full_config = config
        self.visual = Qwen3VLVisionModel(config.vision_config, dtype)
        self.image_token_id = config.image_token_id
        self.video_token_id = getattr(config, "video_token_id", None)
        self.vision_start_token_id = config.vision_start_token_id
        self.spatial_merge_size = getattr(config.vision_config, "spatial_merge_size", 2)
        self.num_deepstack = len(self.visual.deepstack_visual_indexes)

    def _set_mrope_positions(self, input_ids, fb: ForwardBatch) -> None:
        if fb.forward_mode.is_extend():
            fb.mrope_positions = self._extend_positions(input_ids, fb)
        elif fb.mrope_positions is None:
            pos = fb.positions if fb.mrope_position_deltas is None else fb.positions + fb.mrope_position_deltas
            fb.mrope_positions = pos.unsqueeze(0).expand(3, -1).contiguous()

    def _vision_embeds(self, input_ids, fb: ForwardBatch):
        """(input embeddings with the image features in place, per-level deepstack embeddings) — or
        (None, None) when the batch carries no image."""
        if fb.pixel_values is None or fb.image_grid_thw is None or fb.forward_mode.is_decode():
            return None, None
        sync = bool(getattr(fb, "benchmark_vision_timing", False)) and input_ids.is_cuda
        if sync:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        feats = self.visual(fb.pixel_values, fb.image_grid_thw)
        if sync:
            torch.cuda.synchronize()
        fb.vit_prefill_ms = (time.perf_counter() - t0) * 1e3
        mask = input_ids == self.image_token_id
        if self.video_token_id is not None:
            mask = mask | (input_ids == self.video_token_id)
        n_tok = int(mask.sum())
        fb.vit_prefill_tokens = n_tok
        if n_tok != feats.shape[0]:
            raise ValueError(f"Image features and image tokens do not match, tokens: {n_tok}, features: {feats.shape[0]}")
        input_embeds = self.model.embed_tokens(input_ids)
        where = mask.nonzero(as_tuple=True)[0]
        input_embeds.index_copy_(0, where, feats[:, : self.hidden_size].to(input_embeds.dtype))
        deepstack = None
        if self.num_deepstack:
            deepstack = []
            for j in range(self.num_deepstack):
                d = torch.zeros_like(input_embeds)
                d.index_copy_(0, where, feats[:, self.hidden_size * (j + 1): self.hidden_size * (j + 2)].to(d.dtype))
                deepstack.append(d)
        return input_embeds, deepstack

    @staticmethod
    def _visual_name(name: str) -> Optional[str]:
        for pre in ("model.visual.", "visual."):
            if name.startswith(pre):
                return name[len(pre):]
        return None

    def _load_visual(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        """Loads the vision tower's tensors; returns (names loaded, the remaining (name, tensor) pairs)."""
        vparams = {n: p for n, p in self.visual.named_parameters()}
        loaded, rest = set(), []
        for name, tensor in weights:
            vn = self._visual_name(name)
            if vn is None:
                rest.append((name, tensor))
                continue
            # reference checkpoints converted for pymllm use qkv_proj / out_proj for the attention weights
            vn = vn.replace(".attn.qkv_proj.", ".attn.qkv.").replace(".attn.out_proj.", ".attn.proj.")
            p = vparams.get(vn)
            if p is None:
                continue
            p.data.copy_(tensor.reshape(p.shape) if tensor.numel() == p.numel() else tensor)
            loaded.add("visual." + vn)
        return loaded, rest

    def _extend_positions(self, input_ids, fb: ForwardBatch) -> torch.Tensor:
        lens = fb.extend_seq_lens_cpu if getattr(fb, "extend_seq_lens_cpu", None) is not None else fb.extend_seq_lens.tolist()
        prefix = fb.extend_prefix_lens_cpu if getattr(fb, "extend_prefix_lens_cpu", None) is not None else (
            fb.extend_prefix_lens.tolist() if fb.extend_prefix_lens is not None else [0] * len(lens))
        known = fb.mrope_position_deltas.tolist() if fb.mrope_position_deltas is not None else [0] * len(lens)
        grids = None if fb.image_grid_thw is None else fb.image_grid_thw.tolist()
        scales = None if getattr(fb, "mrope_t_scale", None) is None else fb.mrope_t_scale.tolist()
        ids_cpu = input_ids.cpu()
        out, deltas, off, img = [], [], 0, 0
        for i, n in enumerate(lens):
            seq = ids_cpu[off:off + n]
            n_img = int((seq == self.vision_start_token_id).sum())
            thw = grids[img:img + n_img] if (grids is not None and n_img) else None
            ts = scales[img:img + n_img] if (scales is not None and thw is not None) else None
            img += n_img if thw is not None else 0
            p, d = get_rope_index(seq, thw, self.image_token_id, self.vision_start_token_id, self.spatial_merge_size,
                                  start=int(prefix[i]) + int(known[i]), t_scales=ts)
            out.append(p)
            deltas.append(int(known[i]) + d)
            off += n
        fb.mrope_position_deltas = torch.tensor(deltas, dtype=torch.int64, device=input_ids.device)
        return torch.cat(out, 1).to(input_ids.device)


class Qwen3VLForConditionalGeneration(VisionLanguageMixin, Qwen3ForCausalLM):
    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None) -> None:
        tc = _text_config(config)
        rs = getattr(tc, "rope_scaling", None) or getattr(tc, "rope_parameters", None) or {}
        if not isinstance(rs, dict):
            rs = vars(rs)
        sections = rs.get("mrope_section", [24, 20, 20])
        interleaved = bool(rs.get("mrope_interleaved", True))
        if not hasattr(tc, "tie_word_embeddings"):
            tc.tie_word_embeddings = bool(getattr(config, "tie_word_embeddings", False))
        super().__init__(tc, quant_config, params_dtype, mrope_sections=sections, mrope_interleaved=interleaved)
        self._init_vision(config, params_dtype or torch.get_default_dtype())
        self.hidden_size = tc.hidden_size

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, forward_batch: ForwardBatch,
                input_embeds: Optional[torch.Tensor] = None) -> LogitsProcessorOutput:
        fb = forward_batch
        self._set_mrope_positions(input_ids, fb)
        embeds, deepstack = self._vision_embeds(input_ids, fb)
        if embeds is not None:
            input_embeds = embeds
        t0 = time.perf_counter()
        hidden = self.model(input_ids, positions, fb, input_embeds, deepstack_embeds=deepstack)
        out = LogitsProcessorOutput(next_token_logits=self.compute_logits(hidden, fb))
        ms = (time.perf_counter() - t0) * 1e3
        if fb.forward_mode.is_decode():
            fb.llm_decode_ms = ms
        else:
            fb.llm_prefill_ms = ms
        return out

    # ------------------------------------------------------------------ loading
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        loaded, rest = self._load_visual(weights)
        return loaded | super().load_weights(rest)


EntryClass = Qwen3VLForConditionalGeneration

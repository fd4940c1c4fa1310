"""Qwen2-VL (``Qwen2VLForConditionalGeneration``; the reference's C++ runtime has it as ``mllm/models/qwen2vl``): a Qwen2 decoder (q / k / v biases, no q/k norm) with
sectioned — not interleaved — 3-D rotary positions, behind a vision tower that is the Qwen3-VL tower
without the learned position table and without deepstack taps (LayerNorm blocks, QuickGELU MLP, 2 x 2
merger).  The checkpoint's names and config fields are translated here; kernels and control flow are
shared with Qwen3-VL (``VisionLanguageMixin``)."""

from __future__ import annotations

from types import SimpleNamespace
from typing import Iterable, Optional, Tuple

import torch

from .llama import Qwen2ForCausalLM
from .qwen3_vl import VisionLanguageMixin

_VISION_RENAMES = ((".mlp.fc1.", ".mlp.linear_fc1."), (".mlp.fc2.", ".mlp.linear_fc2."), ("merger.ln_q.", "merger.norm."),
                   ("merger.mlp.0.", "merger.linear_fc1."), ("merger.mlp.2.", "merger.linear_fc2."))


def _tower_config(vc) -> SimpleNamespace:
    """Qwen2-VL's vision config in the field names of the shared tower."""
    embed = int(vc.embed_dim)
    return SimpleNamespace(
        hidden_size=embed, num_heads=int(vc.num_heads), patch_size=int(vc.patch_size),
        temporal_patch_size=int(getattr(vc, "temporal_patch_size", 2)), spatial_merge_size=int(getattr(vc, "spatial_merge_size", 2)),
        in_channels=int(getattr(vc, "in_channels", 3)), depth=int(vc.depth), intermediate_size=int(embed * vc.mlp_ratio),
        hidden_act=getattr(vc, "hidden_act", "quick_gelu"), out_hidden_size=int(vc.hidden_size), num_position_embeddings=0,
        deepstack_visual_indexes=[], norm_eps=1e-6)


class Qwen2VLForConditionalGeneration(VisionLanguageMixin, Qwen2ForCausalLM):
    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None) -> None:
        tc = getattr(config, "text_config", config)
        rs = getattr(tc, "rope_scaling", None) or getattr(tc, "rope_parameters", None) or {}
        rs = rs if isinstance(rs, dict) else vars(rs)
        if not hasattr(tc, "tie_word_embeddings"):
            tc.tie_word_embeddings = bool(getattr(config, "tie_word_embeddings", False))
        Qwen2ForCausalLM.__init__(self, tc, quant_config, params_dtype, mrope_sections=rs.get("mrope_section", [16, 24, 24]),
                                  mrope_interleaved=False)
        shim = SimpleNamespace(vision_config=_tower_config(config.vision_config), image_token_id=config.image_token_id,
                               video_token_id=getattr(config, "video_token_id", None),
                               vision_start_token_id=config.vision_start_token_id)
        self._init_vision(shim, params_dtype or torch.get_default_dtype())
        self.full_config = config
        self.hidden_size = tc.hidden_size

    def forward(self, input_ids, positions, forward_batch, input_embeds=None):
        fb = forward_batch
        self._set_mrope_positions(input_ids, fb)
        embeds, _ = self._vision_embeds(input_ids, fb)
        return Qwen2ForCausalLM.forward(self, input_ids, positions, fb, embeds if embeds is not None else input_embeds)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        def renamed():
            for name, t in weights:
                if self._visual_name(name) is not None:
                    for old, new in _VISION_RENAMES:
                        name = name.replace(old, new)
                yield name, t

        loaded, rest = self._load_visual(renamed())
        return loaded | Qwen2ForCausalLM.load_weights(self, rest)


EntryClass = Qwen2VLForConditionalGeneration

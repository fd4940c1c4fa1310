"""Image preprocessing for Qwen3-VL without external image libraries.

Mirrors what the HF Qwen2/3-VL image processor produces (which the reference obtains through
``AutoProcessor`` in pymllm/orchestrator/tokenizer_process.py): resize so both sides are multiples
of ``patch * merge`` within a pixel budget, rescale to [0, 1], normalise with mean = std = 0.5,
repeat the frame ``temporal_patch`` times, and flatten into patches ordered so that the ``merge x
merge`` neighbours of one merged token are consecutive: ``[grid_h * grid_w, C * T * P * P]``.
"""

from __future__ import annotations

import math
from typing import Tuple

import torch
import torch.nn.functional as F


CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 32, min_pixels: int = 64 * 32 * 32,
                 max_pixels: int = 16384 * 32 * 32) -> Tuple[int, int]:
    """Closest size with both sides divisible by ``factor`` and the area inside the pixel budget."""
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def preprocess_image(image: torch.Tensor, patch_size: int = 16, merge_size: int = 2, temporal_patch_size: int = 2,
                     min_pixels: int = 64 * 32 * 32, max_pixels: int = 16384 * 32 * 32,
                     mean=0.5, std=0.5) -> Tuple[torch.Tensor, torch.Tensor]:
    """``image``: uint8 ``[H, W, 3]``.  ``mean`` / ``std``: one number or one per channel (Qwen3-VL normalises with
    0.5 / 0.5, Qwen2-VL and Qwen2.5-VL with the CLIP statistics, :data:`CLIP_MEAN` / :data:`CLIP_STD`).
    Returns ``(pixel_values [N, 3*T*P*P] float32, grid_thw [1, 3])``."""
    if image.dim() != 3 or image.shape[-1] != 3:
        raise ValueError("image must be [H, W, 3]")
    H, W = int(image.shape[0]), int(image.shape[1])
    h, w = smart_resize(H, W, patch_size * merge_size, min_pixels, max_pixels)
    x = image.permute(2, 0, 1).unsqueeze(0).float()
    if (h, w) != (H, W):
        x = F.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255)
    mean_t = torch.as_tensor(mean, dtype=torch.float32).reshape(1, -1, 1, 1)
    std_t = torch.as_tensor(std, dtype=torch.float32).reshape(1, -1, 1, 1)
    x = (x / 255.0 - mean_t) / std_t                                       # [1, 3, h, w]
    x = x.repeat(temporal_patch_size, 1, 1, 1)                             # [T, 3, h, w]  (one temporal group)
    gh, gw = h // patch_size, w // patch_size
    m, P, T = merge_size, patch_size, temporal_patch_size
    x = x.reshape(1, T, 3, gh // m, m, P, gw // m, m, P)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                               # [1, gh/m, gw/m, m, m, C, T, P, P]
    pixel_values = x.reshape(gh * gw, 3 * T * P * P).contiguous()
    return pixel_values, torch.tensor([[1, gh, gw]], dtype=torch.int64)


def image_token_count(grid_thw: torch.Tensor, merge_size: int = 2) -> int:
    g = grid_thw.reshape(-1, 3)
    return int((g[:, 0] * (g[:, 1] // merge_size) * (g[:, 2] // merge_size)).sum())

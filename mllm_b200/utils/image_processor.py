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


def preprocess_video(frames: torch.Tensor, patch_size: int = 16, merge_size: int = 2, temporal_patch_size: int = 2,
                     min_pixels: int = 64 * 32 * 32, max_pixels: int = 768 * 32 * 32,
                     mean=0.5, std=0.5) -> Tuple[torch.Tensor, torch.Tensor]:
    """``frames``: uint8 ``[F, H, W, 3]`` (already sampled).  Consecutive groups of ``temporal_patch_size`` frames
    form one temporal patch (the last frame is repeated when F does not divide); every frame is resized like an
    image, with ``min_pixels`` / ``max_pixels`` bounding one frame.  Returns ``(pixel_values [T*gh*gw, 3*tp*P*P]
    float32, grid_thw [[T, gh, gw]])``, rows ordered temporal patch by temporal patch and, inside one, like
    :func:`preprocess_image` — so the rows of one temporal patch are exactly an image of grid ``[1, gh, gw]``."""
    if frames.dim() != 4 or frames.shape[-1] != 3:
        raise ValueError("frames must be [F, H, W, 3]")
    n, H, W = int(frames.shape[0]), int(frames.shape[1]), int(frames.shape[2])
    if n == 0:
        raise ValueError("a video needs at least one frame")
    tp, m, P = temporal_patch_size, merge_size, patch_size
    if n % tp:
        frames = torch.cat([frames, frames[-1:].expand(tp - n % tp, -1, -1, -1)])
    h, w = smart_resize(H, W, P * m, min_pixels, max_pixels)
    x = frames.permute(0, 3, 1, 2).float()
    if (h, w) != (H, W):
        x = F.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255)
    mean_t = torch.as_tensor(mean, dtype=torch.float32).reshape(1, -1, 1, 1)
    std_t = torch.as_tensor(std, dtype=torch.float32).reshape(1, -1, 1, 1)
    x = (x / 255.0 - mean_t) / std_t                                       # [F', 3, h, w]
    T, gh, gw = x.shape[0] // tp, h // P, w // P
    x = x.reshape(T, tp, 3, gh // m, m, P, gw // m, m, P)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                               # [T, gh/m, gw/m, m, m, C, tp, P, P]
    return x.reshape(T * gh * gw, 3 * tp * P * P).contiguous(), torch.tensor([[T, gh, gw]], dtype=torch.int64)


def sample_frame_indices(total_frames: int, source_fps: float, target_fps: float = 2.0, min_frames: int = 4,
                         max_frames: int = 768) -> list:
    """Evenly spaced frame numbers so that the clip is seen at about ``target_fps``, inside the frame budget."""
    if total_frames <= 0:
        return []
    want = int(total_frames / max(source_fps, 1e-6) * target_fps)
    want = max(min(want, max_frames, total_frames), min(min_frames, total_frames))
    if want <= 1:
        return [0]
    return [int(round(i * (total_frames - 1) / (want - 1))) for i in range(want)]


def sample_frame_indices_strided(total_frames: int, source_fps: float, target_fps: float = 2.0, min_frames: int = 4,
                                 max_frames: int = 768, temporal_patch_size: int = 2) -> list:
    """Frame numbers at a constant stride from frame 0 (the sampling of the Qwen2-VL / Qwen2.5-VL video processor):
    about ``target_fps`` frames per second inside the frame budget, a whole number of temporal patches."""
    if total_frames <= 0:
        return []
    tp = max(1, temporal_patch_size)
    cap = (min(max_frames, total_frames) // tp) * tp
    want = total_frames / max(source_fps, 1e-6) * target_fps
    want = int(min(max(want, min_frames), cap, total_frames) // tp) * tp
    if want <= 0:                                    # fewer frames than one temporal patch: keep them all
        return list(range(total_frames))
    step = total_frames / want
    return [int(i * step) for i in range(want)]


def video_timestamps(frame_indices, source_fps: float, temporal_patch_size: int = 2) -> list:
    """Seconds shown in front of each temporal patch: the mean of the times of its first and last frame (the
    frame list is padded with its last entry to a whole number of patches)."""
    idx = list(frame_indices)
    if len(idx) % temporal_patch_size:
        idx += [idx[-1]] * (temporal_patch_size - len(idx) % temporal_patch_size)
    t = [i / max(source_fps, 1e-6) for i in idx]
    return [(t[i] + t[i + temporal_patch_size - 1]) / 2 for i in range(0, len(t), temporal_patch_size)]

"""Per-step batch description handed from the executor to the model
(fields as pymllm/engine/forward_batch.py:38-191)."""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch


class ForwardMode(enum.IntEnum):
    EXTEND = 1   # prefill of new tokens (possibly after a cached prefix)
    DECODE = 2   # one new token per request
    MIXED = 3    # chunked prefill rows and decode rows in one batch
    IDLE = 4     # no rows on this rank; still joins collectives

    def is_extend(self) -> bool:
        return self in (ForwardMode.EXTEND, ForwardMode.MIXED)

    def is_decode(self) -> bool:
        return self == ForwardMode.DECODE

    def is_mixed(self) -> bool:
        return self == ForwardMode.MIXED

    def is_idle(self) -> bool:
        return self == ForwardMode.IDLE


@dataclass
class ForwardBatch:
    forward_mode: ForwardMode
    batch_size: int
    input_ids: torch.Tensor                    # [T]
    req_pool_indices: torch.Tensor             # [B] rows of req_to_token
    seq_lens: torch.Tensor                     # [B] total length incl. the new tokens
    out_cache_loc: torch.Tensor                # [T] KV slot of every new token
    positions: torch.Tensor                    # [T]
    seq_lens_sum: int = 0
    seq_lens_cpu: Optional[torch.Tensor] = None
    max_seq_len: int = 0
    # extend only
    extend_seq_lens: Optional[torch.Tensor] = None     # [B] new tokens per request
    extend_prefix_lens: Optional[torch.Tensor] = None  # [B] cached tokens per request
    extend_start_loc: Optional[torch.Tensor] = None    # [B] first row of each request in input_ids
    extend_seq_lens_cpu: Optional[List[int]] = None
    extend_prefix_lens_cpu: Optional[List[int]] = None
    max_extend_len: int = 0
    # multimodal
    mrope_positions: Optional[torch.Tensor] = None      # [3, T]
    mrope_position_deltas: Optional[torch.Tensor] = None
    pixel_values: Optional[torch.Tensor] = None
    image_grid_thw: Optional[torch.Tensor] = None
    mrope_t_scale: Optional[torch.Tensor] = None        # [grids] temporal position step per grid (None: 1 everywhere)
    # pools
    req_to_token_pool: Any = None
    token_to_kv_pool: Any = None
    attn_backend: Any = None
    # per-request timing stamps written by the model (host wall clock, ms)
    vit_prefill_ms: Optional[float] = None
    vit_prefill_tokens: Optional[int] = None
    llm_prefill_ms: Optional[float] = None
    llm_decode_ms: Optional[float] = None
    benchmark_vision_timing: bool = False
    extra: dict = field(default_factory=dict)

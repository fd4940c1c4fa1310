"""Quantization section of the global config (pymllm/configs/quantization_config.py:9-18)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional


@dataclass
class QuantizationConfig:
    # Weight scheme override: "compressed-tensors", "awq", "awq_marlin", "w8a8", None.
    method: Optional[str] = None
    kv_cache_dtype: Literal["auto", "float16", "bfloat16", "fp8_e4m3", "fp8_e5m2"] = "auto"

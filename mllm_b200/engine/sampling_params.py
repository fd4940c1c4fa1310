"""Per-request sampling parameters (the keys the reference's server builds in
pymllm/server/launch.py ``_build_sampling_params`` and the runner consumes in
pymllm/executor/model_runner.py:1441-1532)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Union


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    stop: Optional[Union[str, List[str]]] = None
    stop_token_ids: Optional[List[int]] = None
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    seed: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> "SamplingParams":
        d = dict(d or {})
        if "max_tokens" in d and "max_new_tokens" not in d:
            d["max_new_tokens"] = d.pop("max_tokens")
        known = {k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None}
        sp = cls(**known)
        sp.verify()
        return sp

    def verify(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError(f"top_k must be -1 (off) or >= 1, got {self.top_k}")
        if self.top_k > (1 << 30):      # larger than any vocabulary: no filter (and keeps the value inside int32)
            self.top_k = -1
        for name in ("temperature", "top_p", "min_p", "repetition_penalty"):
            v = getattr(self, name)
            if v != v or v in (float("inf"), float("-inf")):
                raise ValueError(f"{name} must be a finite number")
        if not 0 <= self.min_p <= 1:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.max_new_tokens < 0:
            raise ValueError(f"max_new_tokens must be >= 0, got {self.max_new_tokens}")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
        if isinstance(self.stop, str):
            self.stop = [self.stop]

    @property
    def is_greedy(self) -> bool:
        return self.temperature < 1e-6 or self.top_k == 1

    @property
    def has_penalties(self) -> bool:
        return self.frequency_penalty != 0 or self.presence_penalty != 0 or self.repetition_penalty != 1.0

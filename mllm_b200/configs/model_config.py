"""Model section of the global config: a thin view over a HF ``PretrainedConfig``.

Mirrors pymllm/configs/model_config.py:9-31: unknown attributes are looked
up on ``hf_config`` so ``cfg.model.hidden_size`` works once a config is loaded.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class ModelConfig:
    hf_config: Optional[Any] = field(default=None, repr=False)

    def __getattr__(self, name: str) -> Any:
        hf = self.__dict__.get("hf_config")
        if hf is not None and hasattr(hf, name):
            return getattr(hf, name)
        where = "no hf_config is loaded" if hf is None else f"{type(hf).__name__} does not define it either"
        raise AttributeError(f"model config: unknown field {name!r} ({where})")

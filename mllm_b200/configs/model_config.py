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
        raise AttributeError(
            f"'{type(self).__name__}' has no attribute '{name}' "
            f"(also not found on hf_config)"
        )

"""Registry of weight-quantisation schemes (pymllm/quantization/quant_config.py:50-203)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, List, Optional, Type


class QuantizationConfig(ABC):
    """Parsed ``quantization_config`` of a checkpoint; hands a linear method to each layer."""

    @abstractmethod
    def get_name(self) -> str: ...

    @classmethod
    @abstractmethod
    def from_config(cls, config: Dict[str, Any]) -> "QuantizationConfig": ...

    @abstractmethod
    def get_quant_method(self, layer: Any, prefix: str = ""): ...

    @classmethod
    def get_min_capability(cls) -> int:
        return 100  # sm_100

    @staticmethod
    def get_config_filenames() -> List[str]:
        return []

    @staticmethod
    def get_from_keys(config: Dict[str, Any], keys: List[str], default: Any = None) -> Any:
        for k in keys:
            if k in config:
                return config[k]
        if default is not None:
            return default
        raise ValueError(f"none of {keys} found in quantization config")


_REGISTRY: Dict[str, Type[QuantizationConfig]] = {}


def register_quantization(name: str) -> Callable[[Type[QuantizationConfig]], Type[QuantizationConfig]]:
    def deco(cls: Type[QuantizationConfig]) -> Type[QuantizationConfig]:
        if name in _REGISTRY and _REGISTRY[name] is not cls:
            raise ValueError(f"quantization method {name!r} already registered")
        _REGISTRY[name] = cls
        return cls

    return deco


def get_quantization_config(name: str) -> Type[QuantizationConfig]:
    from . import methods  # noqa: F401  (registers the built-in schemes)

    if name not in _REGISTRY:
        raise ValueError(f"unknown quantization method {name!r}; registered: {sorted(_REGISTRY)}")
    return _REGISTRY[name]


def list_quantization_methods() -> List[str]:
    from . import methods  # noqa: F401

    return sorted(_REGISTRY)

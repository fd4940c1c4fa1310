"""Architecture-name -> model-class registry with lazy imports (pymllm/models/__init__.py:19-66)."""

from __future__ import annotations

import importlib
from typing import Dict, Tuple, Type

_REGISTRY: Dict[str, Tuple[str, str]] = {
    "Qwen3ForCausalLM": ("mllm_b200.models.qwen3", "Qwen3ForCausalLM"),
    "Qwen3MoeForCausalLM": ("mllm_b200.models.qwen3_moe", "Qwen3MoeForCausalLM"),
    "Qwen3VLForConditionalGeneration": ("mllm_b200.models.qwen3_vl", "Qwen3VLForConditionalGeneration"),
    "Qwen3VLMoeForConditionalGeneration": ("mllm_b200.models.qwen3_vl_moe", "Qwen3VLMoeForConditionalGeneration"),
    "Qwen3_5ForCausalLM": ("mllm_b200.models.qwen3_5", "Qwen3_5ForCausalLM"),
    "Qwen3_5ForConditionalGeneration": ("mllm_b200.models.qwen3_5", "Qwen3_5ForConditionalGeneration"),
    "Qwen3_5MoeForCausalLM": ("mllm_b200.models.qwen3_5_moe", "Qwen3_5MoeForCausalLM"),
    "Qwen3_5MoeForConditionalGeneration": ("mllm_b200.models.qwen3_5_moe", "Qwen3_5MoeForConditionalGeneration"),
    "Qwen3NextForCausalLM": ("mllm_b200.models.qwen3_next", "Qwen3NextForCausalLM"),
    "LlamaForCausalLM": ("mllm_b200.models.llama", "LlamaForCausalLM"),
    "MistralForCausalLM": ("mllm_b200.models.llama", "MistralForCausalLM"),
    "Qwen2ForCausalLM": ("mllm_b200.models.llama", "Qwen2ForCausalLM"),
    "Qwen2VLForConditionalGeneration": ("mllm_b200.models.qwen2_vl", "Qwen2VLForConditionalGeneration"),
    "Qwen2_5_VLForConditionalGeneration": ("mllm_b200.models.qwen2_5_vl", "Qwen2_5_VLForConditionalGeneration"),
    "Qwen2MoeForCausalLM": ("mllm_b200.models.moe_families", "Qwen2MoeForCausalLM"),
    "MixtralForCausalLM": ("mllm_b200.models.moe_families", "MixtralForCausalLM"),
    "SmolLM3ForCausalLM": ("mllm_b200.models.llama", "SmolLM3ForCausalLM"),
    "MiniCPMForCausalLM": ("mllm_b200.models.minicpm", "MiniCPMForCausalLM"),
    "MiniCPM4ForCausalLM": ("mllm_b200.models.minicpm", "MiniCPMForCausalLM"),
}


def register_model(arch: str, module: str, cls: str) -> None:
    _REGISTRY[arch] = (module, cls)


def supported_architectures():
    return sorted(_REGISTRY)


def get_model_class(arch: str) -> Type:
    if arch not in _REGISTRY:
        raise ValueError(f"Unsupported architecture {arch!r}; supported: {supported_architectures()}")
    module, cls = _REGISTRY[arch]
    return getattr(importlib.import_module(module), cls)

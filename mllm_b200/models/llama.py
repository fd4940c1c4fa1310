"""Llama-family and Qwen2-family decoders (architectures the reference's C++ runtime ships beside Qwen3:
``mllm/models/llama``, ``mllm/models/qwen2_5``, ``mllm/models/smollm3_3B``).  Both are the Qwen3 decoder stack
without the per-head q/k RMSNorm: same fused QKV + RoPE + KV-write prologue (norm weights absent), same
attention and SwiGLU kernels, same tensor-parallel sharding and quantised linears.

* ``LlamaForCausalLM`` (also Mistral-style configs; a ``sliding_window`` is honoured, on fallback attention
  paths): no attention bias unless
  ``attention_bias``; ``rope_scaling`` of type ``llama3`` / ``linear`` / ``yarn`` / ``longrope`` is applied to
  the rotary frequencies (and, for the last two, to the softmax scale).
* ``Qwen2ForCausalLM`` (Qwen2 / Qwen2.5): bias on the q, k and v projections.
* ``SmolLM3ForCausalLM``: Llama with ``no_rope_layers`` — every n-th layer attends without positional
  rotation (the prologue kernel gets all-zero frequencies there).
"""

from __future__ import annotations

from typing import Optional

import torch

from .qwen3 import Qwen3ForCausalLM


def _unsupported(config, what: str, ok) -> None:
    v = getattr(config, what, None)
    if v is not None and not ok(v):
        raise NotImplementedError(f"{type(config).__name__}.{what}={v!r} is not supported")


class LlamaForCausalLM(Qwen3ForCausalLM):
    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None, **model_kw) -> None:
        config.use_qk_norm = False
        if getattr(config, "attention_bias", None) is None:
            config.attention_bias = False
        _unsupported(config, "mlp_bias", lambda v: not v)
        super().__init__(config, quant_config, params_dtype, **model_kw)


class Qwen2ForCausalLM(Qwen3ForCausalLM):
    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None, **model_kw) -> None:
        config.use_qk_norm = False
        config.attention_bias = True          # Qwen2 always has q/k/v biases; the config does not say so
        super().__init__(config, quant_config, params_dtype, **model_kw)


class SmolLM3ForCausalLM(LlamaForCausalLM):
    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None, **model_kw) -> None:
        if getattr(config, "no_rope_layers", None) is None:
            n = int(getattr(config, "no_rope_layer_interval", 4))
            config.no_rope_layers = [int((i + 1) % n != 0) for i in range(config.num_hidden_layers)]
        super().__init__(config, quant_config, params_dtype, **model_kw)


MistralForCausalLM = LlamaForCausalLM
EntryClass = LlamaForCausalLM

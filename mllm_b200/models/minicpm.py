"""MiniCPM / MiniCPM4 decoders (``mllm/models/minicpm4/modeling_minicpm4.hpp``): a Llama stack with three
width/depth-transfer constants and, in MiniCPM4, ``longrope`` rotary scaling.

* the token embeddings are multiplied by ``scale_emb``;
* every block adds ``scale_depth / sqrt(num_hidden_layers)`` times its attention / MLP output to the residual
  stream;
* the final hidden state is divided by ``hidden_size / dim_model_base`` before the output projection.

The residual factor is folded into the ``o_proj`` / ``down_proj`` weights (or their quantisation scales) and the
logit divisor into the final norm weight while the checkpoint is read, so the decoder runs the same fused
add+RMSNorm, GEMM and attention kernels as Llama with no extra pass over the activations; only the embedding
factor is applied at run time (the table may be shared with the output projection, which must stay unscaled).
``longrope``: per-frequency factors in the rotary table, its attention factor in the softmax scale.
"""

from __future__ import annotations

import math
from typing import Iterable, Optional, Tuple

import torch

from .llama import LlamaForCausalLM
from .qwen3 import Qwen3Model

_FLOAT = (torch.float16, torch.bfloat16, torch.float32)
_SCALED_SUFFIXES = (".weight", ".weight_scale", ".weight_scale_inv", ".scales")


class MiniCPMModel(Qwen3Model):
    def forward(self, input_ids, positions, forward_batch, input_embeds=None, deepstack_embeds=None):
        scale = float(getattr(self.config, "scale_emb", 1.0) or 1.0)
        if input_embeds is None and scale != 1.0 and not isinstance(self.embed_tokens, torch.nn.Identity):
            from ..parallel import state as pstate

            if pstate.get_pipeline_parallel_world_size() == 1 or pstate.pp_is_first_stage():
                input_embeds = self.embed_tokens(input_ids) * scale
        return super().forward(input_ids, positions, forward_batch, input_embeds, deepstack_embeds)


class MiniCPMForCausalLM(LlamaForCausalLM):
    model_cls = MiniCPMModel

    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None, **model_kw) -> None:
        super().__init__(config, quant_config, params_dtype, **model_kw)
        self.residual_scale = float(getattr(config, "scale_depth", 1.0) or 1.0) / math.sqrt(config.num_hidden_layers)
        base = float(getattr(config, "dim_model_base", 0) or 0)
        self.logit_divisor = config.hidden_size / base if base > 0 else 1.0

    def _folded(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        for raw, t in weights:
            name = self._canonical_name(raw) or ""
            if (".o_proj" in name or ".down_proj" in name) and name.endswith(_SCALED_SUFFIXES):
                t = torch.as_tensor(t) if not isinstance(t, torch.Tensor) else t
                if t.dtype in _FLOAT and self.residual_scale != 1.0:
                    # every supported format multiplies the stored integers / fp8 values by these tensors
                    t = (t.float() * self.residual_scale).to(t.dtype)
            elif name == "model.norm.weight" and self.logit_divisor != 1.0:
                t = (t.float() / self.logit_divisor).to(t.dtype)
            yield raw, t

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        return super().load_weights(self._folded(weights))


MiniCPM4ForCausalLM = MiniCPMForCausalLM
EntryClass = MiniCPMForCausalLM

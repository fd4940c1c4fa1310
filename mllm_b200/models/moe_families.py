"""Two more mixture-of-experts decoders on the Qwen3-MoE machinery (router kernel, device-side sort,
grouped tcgen05 expert GEMMs, tensor / expert / pipeline parallelism):

* ``Qwen2MoeForCausalLM``: Qwen2 attention (q / k / v biases, no q/k norm); routed experts without
  renormalisation of the top-k weights by default, plus a shared expert scaled by a per-token sigmoid gate.
* ``MixtralForCausalLM``: Llama attention; top-2 of 8 experts, weights renormalised; checkpoints name the
  block ``block_sparse_moe`` and the expert matrices ``w1`` (gate), ``w3`` (up), ``w2`` (down).
"""

from __future__ import annotations

from typing import Iterable, Optional, Tuple

import torch

from ..layers import MLP
from ..layers.moe import SparseMoeBlock
from .qwen3 import Qwen3DecoderLayer, Qwen3Model
from .qwen3_5_moe import SharedExpertMoE
from .qwen3_moe import Qwen3MoeForCausalLM, is_sparse_layer


class _SharedExpertAdapter(SharedExpertMoE):
    """Parameter names of the Qwen3 stack: the layer's MLP prefix is ``model.layers.N.mlp``."""


class Qwen2MoeDecoderLayer(Qwen3DecoderLayer):
    def _make_mlp(self, config, layer_id, quant_config, prefix, params_dtype):
        if not is_sparse_layer(config, layer_id):
            return MLP(config.hidden_size, config.intermediate_size, quant_config, prefix, params_dtype)
        return _SharedExpertAdapter(config, layer_id, quant_config, params_dtype, reduce_results=False)


class Qwen2MoeModel(Qwen3Model):
    layer_cls = Qwen2MoeDecoderLayer


class Qwen2MoeForCausalLM(Qwen3MoeForCausalLM):
    model_cls = Qwen2MoeModel

    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None, **model_kw) -> None:
        config.use_qk_norm = False
        config.attention_bias = True
        if getattr(config, "norm_topk_prob", None) is None:
            config.norm_topk_prob = False
        super().__init__(config, quant_config, params_dtype, **model_kw)


class MixtralForCausalLM(Qwen3MoeForCausalLM):
    _RENAMES = ((".block_sparse_moe.", ".mlp."), (".w1.", ".gate_proj."), (".w3.", ".up_proj."), (".w2.", ".down_proj."))

    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None, **model_kw) -> None:
        config.use_qk_norm = False
        if getattr(config, "attention_bias", None) is None:
            config.attention_bias = False
        config.num_experts = int(getattr(config, "num_local_experts", getattr(config, "num_experts", 8)))
        config.moe_intermediate_size = int(config.intermediate_size)
        config.norm_topk_prob, config.decoder_sparse_step, config.mlp_only_layers = True, 1, []
        super().__init__(config, quant_config, params_dtype, **model_kw)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        def renamed():
            for name, t in weights:
                if ".block_sparse_moe." in name:
                    for old, new in self._RENAMES:
                        name = name.replace(old, new)
                yield name, t

        return super().load_weights(renamed())


EntryClass = Qwen2MoeForCausalLM

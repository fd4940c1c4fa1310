"""Qwen3-Next (``Qwen3NextForCausalLM``): the predecessor layout of the Qwen3.5-MoE hybrid decoder — gated
delta net + gated attention token mixers, routed experts with a gated shared expert (dense MLP on the
layers ``mlp_only_layers`` / ``decoder_sparse_step`` exclude), plain 1-D rotary positions.

Its checkpoints fuse the delta-net input projections per key head:

    in_proj_qkvz rows, for every key head:  [ q (Dk) | k (Dk) | v (rep x Dv) | z (rep x Dv) ]
    in_proj_ba   rows, for every key head:  [ b (rep) | a (rep) ]          rep = value heads per key head

The loader regroups them into the ``[all q | all k | all v]``, ``z``, ``b`` and ``a`` matrices of this
build's delta-net layer (value head ``j`` belongs to key head ``j // rep`` in both layouts), after which
everything is the Qwen3.5-MoE model."""

from __future__ import annotations

from typing import Iterable, Optional, Tuple

import torch

from ..layers import MLP
from .qwen3_5_moe import Qwen3_5MoeDecoderLayer, Qwen3_5MoeForCausalLM, Qwen3_5MoeModel, SharedExpertMoE


def _is_sparse(config, layer_id: int) -> bool:
    return (layer_id not in (getattr(config, "mlp_only_layers", None) or [])
            and int(getattr(config, "num_experts", 0)) > 0
            and (layer_id + 1) % max(1, int(getattr(config, "decoder_sparse_step", 1))) == 0)


class Qwen3NextDecoderLayer(Qwen3_5MoeDecoderLayer):
    def _make_mlp(self, config, layer_id, quant_config, params_dtype):
        if _is_sparse(config, layer_id):
            return SharedExpertMoE(config, layer_id, quant_config, params_dtype)
        return MLP(config.hidden_size, config.intermediate_size, quant_config, f"model.layers.{layer_id}.mlp",
                   params_dtype, reduce_results=True)


class Qwen3NextModel(Qwen3_5MoeModel):
    layer_cls = Qwen3NextDecoderLayer


class Qwen3NextForCausalLM(Qwen3_5MoeForCausalLM):
    model_cls = Qwen3NextModel

    def _regroup(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        c = self.config
        hk, hv = int(c.linear_num_key_heads), int(c.linear_num_value_heads)
        dk, dv = int(c.linear_key_head_dim), int(c.linear_value_head_dim)
        rep = hv // hk
        for name, t in weights:
            if name.endswith("linear_attn.in_proj_qkvz.weight"):
                base = name[: -len("in_proj_qkvz.weight")]
                full = t.materialize() if hasattr(t, "materialize") else t
                w = full.reshape(hk, 2 * dk + 2 * rep * dv, full.shape[-1])
                q, k = w[:, :dk], w[:, dk:2 * dk]
                v, z = w[:, 2 * dk:2 * dk + rep * dv], w[:, 2 * dk + rep * dv:]
                flat = lambda x: x.reshape(-1, full.shape[-1])  # noqa: E731
                yield base + "in_proj_qkv.weight", torch.cat([flat(q), flat(k), flat(v)], 0)
                yield base + "in_proj_z.weight", flat(z).contiguous()
            elif name.endswith("linear_attn.in_proj_ba.weight"):
                base = name[: -len("in_proj_ba.weight")]
                full = t.materialize() if hasattr(t, "materialize") else t
                w = full.reshape(hk, 2 * rep, full.shape[-1])
                yield base + "in_proj_b.weight", w[:, :rep].reshape(hv, -1).contiguous()
                yield base + "in_proj_a.weight", w[:, rep:].reshape(hv, -1).contiguous()
            else:
                yield name, t

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        return super().load_weights(self._regroup(weights))


EntryClass = Qwen3NextForCausalLM

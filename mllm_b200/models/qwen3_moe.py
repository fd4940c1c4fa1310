"""Qwen3-MoE (Qwen3MoeForCausalLM): the Qwen3 decoder with sparse MoE MLPs.

The reference ships no GPU implementation (``pymllm/models/qwen3_moe.py`` is an empty file); the
semantics come from its C++ CPU model (mllm/models/qwen3_moe/modeling_qwen3_moe_fa2.hpp:71-373):
a layer is sparse iff it is not listed in ``mlp_only_layers``, ``num_experts > 0`` and
``(layer + 1) % decoder_sparse_step == 0``; otherwise it uses the dense MLP of width
``intermediate_size``.  Checkpoint names are the HF ones
(``mlp.gate.weight``, ``mlp.experts.E.{gate,up,down}_proj.weight``).
"""

from __future__ import annotations

import re
from typing import Iterable, Optional, Tuple

import torch

from ..layers import MLP
from ..layers.moe import SparseMoeBlock
from ..parallel import state as pstate
from .qwen3 import Qwen3DecoderLayer, Qwen3ForCausalLM, Qwen3Model

_EXPERT_RE = re.compile(r"^(.*\.mlp)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
# newer checkpoints keep all experts of a layer in two 3-D tensors
_FUSED_EXPERT_RE = re.compile(r"^(.*\.mlp)\.experts\.(gate_up_proj|down_proj)$")


def is_sparse_layer(config, layer_id: int) -> bool:
    return (layer_id not in (getattr(config, "mlp_only_layers", None) or [])
            and getattr(config, "num_experts", 0) > 0
            and (layer_id + 1) % max(1, getattr(config, "decoder_sparse_step", 1)) == 0)


class _MoEMlp(torch.nn.Module):
    """Adapter giving SparseMoeBlock the calling convention of the dense MLP."""

    def __init__(self, block: SparseMoeBlock) -> None:
        super().__init__()
        self.block = block
        self.gate = block.gate  # so that ``mlp.gate.weight`` loads by name

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.block(x)
        if not isinstance(y, torch.Tensor):
            return y            # this rank's rows, complete (expert-parallel exchange): the next norm takes it as is
        tp = pstate.get_tensor_model_parallel_world_size()
        if tp > 1 and not self.block.is_partial:
            # every rank computed the full output: keep one copy in the sum that the next norm reduces
            return y if pstate.get_tensor_model_parallel_rank() == 0 else torch.zeros_like(y)
        return y


class Qwen3MoeDecoderLayer(Qwen3DecoderLayer):
    def _make_mlp(self, config, layer_id, quant_config, prefix, params_dtype):
        if not is_sparse_layer(config, layer_id):
            return MLP(config.hidden_size, config.intermediate_size, quant_config, prefix, params_dtype)
        block = SparseMoeBlock(config.hidden_size, config.moe_intermediate_size, config.num_experts,
                               config.num_experts_per_tok, bool(getattr(config, "norm_topk_prob", True)),
                               params_dtype, prefix)
        return _MoEMlp(block)


class Qwen3MoeModel(Qwen3Model):
    layer_cls = Qwen3MoeDecoderLayer


class Qwen3MoeForCausalLM(Qwen3ForCausalLM):
    model_cls = Qwen3MoeModel

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        params = dict(self.named_parameters())
        rest = []
        loaded = set()
        for name, tensor in self._split_fused_experts(self._dequantized_experts(weights)):
            canon = self._canonical_name(name)
            m = _EXPERT_RE.match(canon) if canon else None
            if m is None:
                if canon is not None and canon.endswith(".mlp.gate.weight"):
                    # router weight lives on the block's gate module
                    target = canon.replace(".mlp.gate.weight", ".mlp.block.gate.weight")
                    if target in params:
                        params[target].data.copy_(tensor)
                        loaded.add(target)
                        continue
                rest.append((name, tensor))
                continue
            prefix, expert, which = m.group(1), int(m.group(2)), m.group(3)
            if which == "down_proj":
                p = params.get(f"{prefix}.block.w2")
                if p is not None:
                    p.weight_loader(p, tensor, expert)
                    loaded.add(f"{prefix}.block.w2")
            else:
                p = params.get(f"{prefix}.block.w13")
                if p is not None:
                    p.weight_loader(p, tensor, expert, "gate" if which == "gate_proj" else "up")
                    loaded.add(f"{prefix}.block.w13")
        loaded |= super().load_weights(rest)
        return loaded

    def _dequantized_experts(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        from ..quantization.expert_dequant import dequantized_experts

        return dequantized_experts(weights, self.quant_config, self.model.embed_tokens.weight.dtype)

    def _split_fused_experts(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        """Yields per-expert ``gate_proj`` / ``up_proj`` / ``down_proj`` matrices for checkpoints that store
        ``experts.gate_up_proj`` ``[E, 2I, H]`` (or ``[E, H, 2I]``) and ``experts.down_proj`` ``[E, H, I]``
        (or ``[E, I, H]``); everything else passes through."""
        tc = self.config
        inter, hidden = int(getattr(tc, "moe_intermediate_size", 0)), int(tc.hidden_size)
        for name, tensor in weights:
            m = _FUSED_EXPERT_RE.match(self._canonical_name(name) or "")
            if m is None or tensor.dim() != 3:
                yield name, tensor
                continue
            base = name[: name.rindex(".experts.") + len(".experts.")]
            t = tensor.materialize() if hasattr(tensor, "materialize") else tensor
            for e in range(t.shape[0]):
                w = t[e]
                if m.group(2) == "gate_up_proj":
                    w = w if w.shape[0] == 2 * inter else w.t()
                    yield f"{base}{e}.gate_proj.weight", w[:inter]
                    yield f"{base}{e}.up_proj.weight", w[inter:]
                else:
                    yield f"{base}{e}.down_proj.weight", (w if w.shape[0] == hidden else w.t())

    def post_load(self) -> None:
        for m in self.modules():
            if isinstance(m, SparseMoeBlock):
                m.process_weights_after_loading()


EntryClass = Qwen3MoeForCausalLM

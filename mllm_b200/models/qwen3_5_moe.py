"""Qwen3.5 mixture-of-experts models (``Qwen3_5MoeForCausalLM`` / ``Qwen3_5MoeForConditionalGeneration``):
the hybrid decoder of Qwen3.5 (gated delta net + gated attention layers) whose feed-forward block is, in
every layer, routed experts plus one always-on shared expert scaled by a per-token sigmoid gate:

    y = experts(x; top-k of softmax(router(x)), renormalised) + sigmoid(x . g) * shared_mlp(x)

The routed part is the same ``SparseMoeBlock`` as Qwen3-MoE (router kernel, device-side sort, grouped
tcgen05 GEMMs; tensor- or expert-parallel); under tensor parallelism the routed partial sums and the
shared expert's partial sums are added first and reduced once.
"""

from __future__ import annotations

import re
from typing import Iterable, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..layers import MLP
from ..layers.moe import SparseMoeBlock
from ..parallel import state as pstate
from .qwen3_5 import Qwen3_5DecoderLayer, Qwen3_5ForCausalLM, Qwen3_5ForConditionalGeneration, Qwen3_5Model

_EXPERT_RE = re.compile(r"^(.*\.mlp)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
_FUSED_RE = re.compile(r"^(.*\.mlp)\.experts\.(gate_up_proj|down_proj)$")
_PREFIXES = (("model.language_model.", "model."), ("language_model.model.", "model."), ("language_model.", "model."))


class SharedExpertMoE(nn.Module):
    """``reduce_results=False`` leaves this rank's partial sums for the caller (decoder stacks whose next
    norm performs the tensor-parallel reduction)."""

    def __init__(self, config, layer_id: int, quant_config=None, params_dtype=None, reduce_results: bool = True) -> None:
        super().__init__()
        self.reduce_results = reduce_results
        prefix = f"model.layers.{layer_id}.mlp"
        dt = params_dtype or torch.get_default_dtype()
        self.block = SparseMoeBlock(config.hidden_size, config.moe_intermediate_size, config.num_experts,
                                    config.num_experts_per_tok, bool(getattr(config, "norm_topk_prob", True)), dt, prefix)
        self.gate = self.block.gate                      # ``mlp.gate.weight`` is the router
        self.shared_expert = MLP(config.hidden_size, config.shared_expert_intermediate_size, quant_config,
                                 f"{prefix}.shared_expert", dt, reduce_results=False)
        self.shared_expert_gate = nn.Module()
        self.shared_expert_gate.weight = nn.Parameter(torch.zeros(1, config.hidden_size, dtype=dt), requires_grad=False)
        self.tp = pstate.get_tensor_model_parallel_world_size()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        routed = self.block(x)
        if self.tp > 1 and not self.block.is_partial and pstate.get_tensor_model_parallel_rank() != 0:
            routed = torch.zeros_like(routed)            # every rank holds the full routed output: count it once
        shared = self.shared_expert(x)                   # a partial sum under tensor parallelism
        g = torch.sigmoid(torch.nn.functional.linear(x.float(), self.shared_expert_gate.weight.float())).to(x.dtype)
        y = routed + g * shared
        return pstate.tensor_model_parallel_all_reduce(y) if self.tp > 1 and self.reduce_results else y


class Qwen3_5MoeDecoderLayer(Qwen3_5DecoderLayer):
    def _make_mlp(self, config, layer_id, quant_config, params_dtype):
        return SharedExpertMoE(config, layer_id, quant_config, params_dtype)


class Qwen3_5MoeModel(Qwen3_5Model):
    layer_cls = Qwen3_5MoeDecoderLayer


class _MoeLoading:
    """Expert tensors (one matrix per expert, or all experts of a layer fused in two 3-D tensors) go to the
    routed block; everything else to the hybrid model's loader."""

    def _load_moe(self, weights: Iterable[Tuple[str, torch.Tensor]], base_loader) -> set:
        params = dict(self.named_parameters())
        inter, hidden = int(self.config.moe_intermediate_size), int(self.config.hidden_size)
        loaded, rest = set(), []

        def put(prefix: str, expert: int, which: str, w: torch.Tensor) -> None:
            if which == "down_proj":
                p = params.get(f"{prefix}.block.w2")
                if p is not None:
                    p.weight_loader(p, w, expert)
                    loaded.add(f"{prefix}.block.w2")
            else:
                p = params.get(f"{prefix}.block.w13")
                if p is not None:
                    p.weight_loader(p, w, expert, "gate" if which == "gate_proj" else "up")
                    loaded.add(f"{prefix}.block.w13")

        from ..quantization.expert_dequant import dequantized_experts

        for name, t in dequantized_experts(weights, getattr(self, "quant_config", None), self.model.embed_tokens.weight.dtype):
            canon = name
            for old, new in _PREFIXES:
                if canon.startswith(old):
                    canon = new + canon[len(old):]
                    break
            m = _EXPERT_RE.match(canon)
            if m is not None:
                put(m.group(1), int(m.group(2)), m.group(3), t)
                continue
            m = _FUSED_RE.match(canon)
            if m is not None and t.dim() == 3:
                full = t.materialize() if hasattr(t, "materialize") else t
                for e in range(full.shape[0]):
                    w = full[e]
                    if m.group(2) == "gate_up_proj":
                        w = w if w.shape[0] == 2 * inter else w.t()
                        put(m.group(1), e, "gate_proj", w[:inter])
                        put(m.group(1), e, "up_proj", w[inter:])
                    else:
                        put(m.group(1), e, "down_proj", w if w.shape[0] == hidden else w.t())
                continue
            if canon.endswith(".mlp.gate.weight"):
                target = canon.replace(".mlp.gate.weight", ".mlp.block.gate.weight")
                if target in params:
                    params[target].data.copy_(t)
                    loaded.update((target, canon))
                    continue
            rest.append((name, t))
        return loaded | base_loader(rest)

    def _post_load_moe(self) -> None:
        for m in self.modules():
            if isinstance(m, SparseMoeBlock):
                m.process_weights_after_loading()


class Qwen3_5MoeForCausalLM(_MoeLoading, Qwen3_5ForCausalLM):
    model_cls = Qwen3_5MoeModel

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        return self._load_moe(weights, lambda rest: Qwen3_5ForCausalLM.load_weights(self, rest))

    def post_load(self) -> None:
        Qwen3_5ForCausalLM.post_load(self)
        self._post_load_moe()


class Qwen3_5MoeForConditionalGeneration(_MoeLoading, Qwen3_5ForConditionalGeneration):
    model_cls = Qwen3_5MoeModel

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        return self._load_moe(weights, lambda rest: Qwen3_5ForConditionalGeneration.load_weights(self, rest))

    def post_load(self) -> None:
        Qwen3_5ForConditionalGeneration.post_load(self)
        self._post_load_moe()


EntryClass = Qwen3_5MoeForCausalLM

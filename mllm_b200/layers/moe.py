"""Sparse mixture-of-experts block (Qwen3-MoE).

Router and expert semantics follow the reference's C++ model
(mllm/models/qwen3_moe/modeling_qwen3_moe_fa2.hpp:71-239): fp32 softmax over all experts, sorted
top-k, optional renormalisation, then for every expert the SwiGLU MLP over its tokens and a
weighted sum over the k choices.  The reference loops over experts on the CPU; here the experts'
weights are stacked (``w13 [E_local, 2I, H]``, ``w2 [E_local, H, I]``), tokens are grouped by expert
and each group runs through the tcgen05 GEMMs (SwiGLU fused into the first one).

Expert parallelism: with ``ep_size > 1`` each rank owns ``E / ep`` consecutive experts; every rank
sees all tokens of the batch (attention is tensor-parallel, activations are replicated), computes
the contribution of its own experts, and the partial outputs are summed by the same fused
reduction that closes every tensor-parallel block.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..parallel import state as pstate


class MoEGate(nn.Module):
    def __init__(self, hidden_size: int, num_experts: int, top_k: int, norm_topk_prob: bool, params_dtype=None) -> None:
        super().__init__()
        self.top_k, self.norm_topk_prob = top_k, norm_topk_prob
        self.weight = nn.Parameter(torch.empty(num_experts, hidden_size, dtype=params_dtype or torch.get_default_dtype()),
                                   requires_grad=False)

    def forward(self, x: torch.Tensor):
        return ops.moe_router_topk(x, self.weight, self.top_k, self.norm_topk_prob)


class SparseMoeBlock(nn.Module):
    def __init__(self, hidden_size: int, moe_intermediate_size: int, num_experts: int, top_k: int,
                 norm_topk_prob: bool = True, params_dtype=None, prefix: str = "") -> None:
        super().__init__()
        ep = pstate.get_ep_group()
        self.ep_size, self.ep_rank = ep.world_size, ep.rank_in_group
        self.tp_size = pstate.get_tensor_model_parallel_world_size()
        if num_experts % self.ep_size:
            raise ValueError(f"num_experts={num_experts} not divisible by ep_size={self.ep_size}")
        self.num_experts = num_experts
        self.local_experts = num_experts // self.ep_size
        self.expert_offset = self.ep_rank * self.local_experts
        # without expert parallelism the experts' intermediate dimension is tensor-parallel instead
        self.inter_shard = 1 if self.ep_size > 1 else self.tp_size
        self.inter = moe_intermediate_size // self.inter_shard
        dt = params_dtype or torch.get_default_dtype()
        self.gate = MoEGate(hidden_size, num_experts, top_k, norm_topk_prob, dt)
        self.w13 = nn.Parameter(torch.empty(self.local_experts, 2 * self.inter, hidden_size, dtype=dt), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(self.local_experts, hidden_size, self.inter, dtype=dt), requires_grad=False)
        self.w13.weight_loader = self._load_w13
        self.w2.weight_loader = self._load_w2
        self.swiglu_block = 0
        self.prefix = prefix

    # checkpoint names: experts.E.{gate_proj,up_proj,down_proj}.weight
    def owns(self, expert: int) -> bool:
        return self.expert_offset <= expert < self.expert_offset + self.local_experts

    def _shard(self, w: torch.Tensor, dim: int) -> torch.Tensor:
        if self.inter_shard == 1:
            return w
        r = pstate.get_tensor_model_parallel_rank()
        return w.narrow(dim, r * self.inter, self.inter)

    def _load_w13(self, param, loaded: torch.Tensor, expert: int, which: str) -> None:
        if not self.owns(expert):
            return
        e = expert - self.expert_offset
        part = self._shard(loaded, 0)
        off = 0 if which == "gate" else self.inter
        param.data[e, off : off + self.inter].copy_(part)

    def _load_w2(self, param, loaded: torch.Tensor, expert: int, which: str = "down") -> None:
        if not self.owns(expert):
            return
        param.data[expert - self.expert_offset].copy_(self._shard(loaded, 1))

    def process_weights_after_loading(self) -> None:
        """Interleave gate/up rows in blocks of 128 so the first GEMM can fuse the SwiGLU."""
        if self.swiglu_block == 0 and (2 * self.inter) % (2 * ops.SWIGLU_BLOCK) == 0 and self.w13.is_cuda:
            w = self.w13.data
            for e in range(w.shape[0]):
                w[e] = ops.ref.interleave_gate_up(w[e].clone(), ops.SWIGLU_BLOCK)
            self.swiglu_block = ops.SWIGLU_BLOCK

    def forward(self, x: torch.Tensor):
        """Returns this rank's contribution (a partial sum when ``ep_size`` or ``tp_size`` > 1).

        Inside the fused tensor-parallel prefill step (``x`` is the gathered buffer, the residual stream is
        sharded by rows) with the expert-parallel exchange set up, the rank routes only the rows it owns, the
        rows travel to their experts' ranks and back (``ops.ep_moe_exchange``), and the result is a
        ``PrefillShard``: this rank's rows, complete, for the following norm."""
        shard = self._exchange(x)
        if shard is not None:
            return shard
        topk_w, topk_ids = self.gate(x)
        return ops.moe_experts(x, self.w13, self.w2, topk_w, topk_ids, self.expert_offset, self.swiglu_block,
                               self.num_experts)

    def can_exchange(self, rows: int) -> bool:
        """Whether a batch of ``rows`` tokens can go through the expert-parallel exchange on this block."""
        from ..parallel.symm import get_ep_comm, get_tp_comm

        ep, tp = get_ep_comm(), get_tp_comm()
        return (ep is not None and tp is not None and tp.prefill is not None and self.ep_size == ep.world
                and self.swiglu_block == ops.SWIGLU_BLOCK and self.w13.is_cuda and ep.eligible(rows))

    def _exchange(self, x: torch.Tensor):
        from ..parallel.symm import PrefillShard, get_ep_comm, get_tp_comm

        ep, tp = get_ep_comm(), get_tp_comm()
        if (x.dim() != 2 or not x.is_cuda or not self.can_exchange(x.shape[0])
                or x.data_ptr() != tp.prefill.hidden_full.data_ptr()):
            return None
        own = x.shape[0] // ep.world
        mine = x[ep.rank * own:(ep.rank + 1) * own]
        topk_w, topk_ids = self.gate(mine)
        out = ops.ep_moe_exchange(mine, self.w13, self.w2, topk_w, topk_ids, self.swiglu_block, ep)
        return PrefillShard(x.shape[0], tp.next_epoch(), out)

    @property
    def is_partial(self) -> bool:
        return self.ep_size > 1 or self.tp_size > 1

"""RMSNorm / LayerNorm modules over the fused kernels (roles of pymllm/layers/rms_norm.py:64-166
and layer_norm.py:11-43)."""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, params_dtype: Optional[torch.dtype] = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=params_dtype or torch.get_default_dtype()),
                                   requires_grad=False)
        self.eps = eps

    def forward(self, x, residual: Optional[torch.Tensor] = None, partial: bool = False, gated: bool = False
                ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        """Without ``residual``: returns the normed tensor.  With it: in place ``residual += x`` and
        ``x = norm(residual)``; returns ``(x, residual)``.  ``partial=True`` says ``x`` holds this
        tensor-parallel rank's partial sums: the reduction over ranks is fused into the same step.

        When ``x`` is a ``PrefillPartial`` (the row-parallel GEMM scattered its tiles to the owning ranks)
        the step is reduce-scatter + add + norm + all-gather; the returned residual is then this rank's
        row shard, and ``gated=True`` promises that the consumer of the normed rows is a GEMM that waits
        per row tile (otherwise the stream waits for the whole gather here)."""
        from ..parallel.symm import PrefillPartial, PrefillShard, get_tp_comm

        if isinstance(x, (PrefillPartial, PrefillShard)):
            assert residual is not None
            return ops.tp_rs_add_rmsnorm_ag(x, residual, self.weight, self.eps, get_tp_comm(), gated)
        if partial:
            assert residual is not None
            if residual.shape[0] != x.shape[0]:
                raise RuntimeError("row-sharded residual met a full partial sum: fused and plain tensor-parallel "
                                   "steps were mixed inside one forward pass")
            return ops.tp_reduce_add_rmsnorm(x, residual, self.weight, self.eps), residual
        if residual is None:
            return ops.rmsnorm(x, self.weight, self.eps)
        ops.fused_add_rmsnorm(x, residual, self.weight, self.eps)
        return x, residual


class GemmaRMSNorm(RMSNorm):
    """``x * rsqrt(mean x^2 + eps) * (1 + w)``; the offset is folded into the weight at load."""

    def load_offset_weight(self, w: torch.Tensor) -> None:
        self.weight.data.copy_((w.float() + 1.0).to(self.weight.dtype))


class LayerNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, bias: bool = True,
                 params_dtype: Optional[torch.dtype] = None) -> None:
        super().__init__()
        dt = params_dtype or torch.get_default_dtype()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dt), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dt), requires_grad=False) if bias else None
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layernorm(x, self.weight, self.bias, self.eps)

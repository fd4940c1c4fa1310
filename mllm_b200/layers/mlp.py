"""Gated MLP: fused gate/up projection with the SwiGLU folded into the GEMM epilogue, then the
down projection (roles of pymllm/layers/mlp.py:58-231; the tensor-parallel form splits gate/up by
columns and down by rows, one reduction per MLP)."""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .linear import MergedLinear, RowParallelLinear


class MLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, quant_config=None, prefix: str = "",
                 params_dtype: Optional[torch.dtype] = None, reduce_results: bool = False) -> None:
        super().__init__()

        def qm(name):
            return quant_config.get_quant_method(None, f"{prefix}.{name}") if quant_config is not None else None

        self.gate_up_proj = MergedLinear(hidden_size, [intermediate_size, intermediate_size],
                                         quant_method=qm("gate_up_proj"), params_dtype=params_dtype,
                                         prefix=f"{prefix}.gate_up_proj")
        self.gate_up_proj.swiglu_fused = True
        self.down_proj = RowParallelLinear(intermediate_size, hidden_size, quant_method=qm("down_proj"),
                                           params_dtype=params_dtype, prefix=f"{prefix}.down_proj",
                                           reduce_results=reduce_results)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.gate_up_proj.forward_swiglu(x)
        if self.down_proj.tp_size > 1 and not self.down_proj.reduce_results:
            return self.down_proj.forward_partial(h)
        return self.down_proj(h)


ParallelMLP = MLP

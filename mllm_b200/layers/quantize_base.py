"""Plug-in interface between linear layers and weight formats.

A linear layer owns no weight by itself: at construction it asks its
``quant_method`` to ``create_weights`` (registering the parameters the checkpoint
format needs, each tagged with a ``weight_loader``), after loading it calls
``process_weights_after_loading`` (re-layout for the kernels) and at run time
``apply`` (the GEMM).  Same contract as pymllm/layers/quantize_base.py:63-275.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch
from torch import nn

from .. import ops


def set_weight_attrs(param: torch.Tensor, attrs: Optional[Dict[str, Any]]) -> None:
    for k, v in (attrs or {}).items():
        setattr(param, k, v)


class QuantizeMethodBase:
    def create_weights(self, layer: nn.Module, *args, **kwargs) -> None:
        raise NotImplementedError

    def apply(self, layer: nn.Module, *args, **kwargs) -> torch.Tensor:
        raise NotImplementedError

    def process_weights_after_loading(self, layer: nn.Module) -> None:
        return None


class LinearMethodBase(QuantizeMethodBase):
    def create_weights(
        self, layer: nn.Module, input_size_per_partition: int, output_partition_sizes: List[int],
        input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs,
    ) -> None:
        raise NotImplementedError

    def apply(self, layer: nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None,
              residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def apply_swiglu(self, layer: nn.Module, x: torch.Tensor) -> torch.Tensor:
        """Fused gate/up projection + SwiGLU; default = apply then activation."""
        return ops.silu_and_mul(self.apply(layer, x))


class UnquantizedLinearMethod(LinearMethodBase):
    """bf16 / fp16 weights ``[out, in]``; GEMM on tcgen05 (the reference calls ``F.linear``)."""

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra_weight_attrs) -> None:
        w = nn.Parameter(
            torch.empty(sum(output_partition_sizes), input_size_per_partition, dtype=params_dtype),
            requires_grad=False,
        )
        set_weight_attrs(w, {"input_dim": 1, "output_dim": 0})
        set_weight_attrs(w, extra_weight_attrs)
        layer.register_parameter("weight", w)

    def process_weights_after_loading(self, layer) -> None:
        if getattr(layer, "swiglu_fused", False) and not getattr(layer, "_gate_up_interleaved", False):
            w = layer.weight.data
            if w.shape[0] % (2 * ops.SWIGLU_BLOCK) == 0:
                layer.weight.data = ops.ref.interleave_gate_up(w, ops.SWIGLU_BLOCK).contiguous()
                layer._gate_up_interleaved = True

    def apply(self, layer, x, bias=None, residual=None):
        return ops.linear(x, layer.weight, bias, residual)

    def apply_swiglu(self, layer, x):
        if getattr(layer, "_gate_up_interleaved", False):
            return ops.linear_swiglu(x, layer.weight, ops.SWIGLU_BLOCK)
        return ops.silu_and_mul(ops.linear(x, layer.weight))

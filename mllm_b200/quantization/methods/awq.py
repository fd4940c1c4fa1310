"""AutoAWQ checkpoints (``quant_method: "awq"``, served under the name ``awq_marlin`` like the
reference: pymllm/quantization/methods/awq_marlin.py:108-524).

Checkpoint tensors per linear: ``qweight`` int32 ``[K, N/8]``, ``qzeros`` int32 ``[K/g, N/8]`` (both
packed along N in AWQ's interleaved nibble order 0,2,4,6,1,3,5,7) and ``scales`` fp16 ``[K/g, N]``;
``w = (q - z) * s``.  After loading, the tensors are unpacked once and re-laid-out K-major:
``weight_packed`` int32 ``[N, K/8]`` in natural nibble order, ``weight_zeros`` uint8 ``[N, K/g]`` and
``weight_scale`` ``[N, K/g]`` — the operand layout of the tcgen05 W4A16 kernel (the reference repacks
for Marlin instead).
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ... import ops
from ...layers.quantize_base import LinearMethodBase, UnquantizedLinearMethod, set_weight_attrs
from ..quant_config import QuantizationConfig, register_quantization

# position p of a packed AWQ word holds logical column AWQ_ORDER[p]
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def unpack_awq(packed: torch.Tensor) -> torch.Tensor:
    """int32 ``[R, C/8]`` in AWQ nibble order -> uint8-valued ``[R, C]``."""
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    nib = ((packed.unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8)  # [R, C/8, 8] by position
    out = torch.empty_like(nib)
    for pos, col in enumerate(AWQ_ORDER):
        out[..., col] = nib[..., pos]
    return out.reshape(packed.shape[0], -1)


def pack_awq(values: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`unpack_awq` (used by tests and the random-checkpoint writer)."""
    v = values.reshape(values.shape[0], -1, 8).to(torch.int32)
    word = torch.zeros(v.shape[:2], dtype=torch.int32, device=values.device)
    for pos, col in enumerate(AWQ_ORDER):
        word |= (v[..., col] & 0xF) << (4 * pos)
    return word


def pack_rows_natural(values: torch.Tensor) -> torch.Tensor:
    """uint4 values ``[N, K]`` -> int32 ``[N, K/8]`` with nibble i of word j = element 8j+i."""
    v = values.reshape(values.shape[0], -1, 8).to(torch.int64)
    word = torch.zeros(v.shape[:2], dtype=torch.int64, device=values.device)
    for i in range(8):
        word |= (v[..., i] & 0xF) << (4 * i)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


class AWQLinearMethod(LinearMethodBase):
    def __init__(self, group_size: int, zero_point: bool = True) -> None:
        self.group_size = group_size
        self.zero_point = zero_point

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra) -> None:
        n, k = sum(output_partition_sizes), input_size_per_partition
        g = k if self.group_size == -1 else self.group_size
        if n % 8 or k % g:
            raise ValueError(f"AWQ: N={n} must be divisible by 8 and K={k} by the group size {g}")
        qweight = nn.Parameter(torch.zeros(k, n // 8, dtype=torch.int32), requires_grad=False)
        qzeros = nn.Parameter(torch.zeros(k // g, n // 8, dtype=torch.int32), requires_grad=False)
        scales = nn.Parameter(torch.zeros(k // g, n, dtype=params_dtype), requires_grad=False)
        set_weight_attrs(qweight, {"input_dim": 0, "output_dim": 1, "packed_dim": 1, "pack_factor": 8})
        set_weight_attrs(qzeros, {"input_dim": 0, "output_dim": 1, "packed_dim": 1, "pack_factor": 8})
        set_weight_attrs(scales, {"input_dim": 0, "output_dim": 1})
        for p in (qweight, qzeros, scales):
            set_weight_attrs(p, extra)
        layer.register_parameter("qweight", qweight)
        layer.register_parameter("qzeros", qzeros)
        layer.register_parameter("scales", scales)
        layer.w4_group = g

    def process_weights_after_loading(self, layer) -> None:
        if not hasattr(layer, "qweight"):
            return
        q = unpack_awq(layer.qweight.data)              # [K, N]
        z = unpack_awq(layer.qzeros.data)               # [K/g, N]
        packed = pack_rows_natural(q.t().contiguous())  # [N, K/8]
        zeros = z.t().contiguous().to(torch.uint8)      # [N, K/g]
        scale = layer.scales.data.t().contiguous()      # [N, K/g]
        for name in ("qweight", "qzeros", "scales"):
            delattr(layer, name)
        layer.w4_interleaved = packed.is_cuda     # GPU: nibble order the GEMM kernel expands fastest
        if layer.w4_interleaved:
            packed = ops.w4a16_interleave(packed)
        layer.register_parameter("weight_packed", nn.Parameter(packed, requires_grad=False))
        layer.register_parameter("weight_zeros", nn.Parameter(zeros, requires_grad=False))
        layer.register_parameter("weight_scale", nn.Parameter(scale, requires_grad=False))

    def apply(self, layer, x, bias=None, residual=None):
        y = ops.w4a16_gemm(x, layer.weight_packed, layer.weight_scale, layer.weight_zeros, layer.w4_group, bias,
                            interleaved=getattr(layer, "w4_interleaved", False))
        return y if residual is None else y + residual


@register_quantization("awq_marlin")
class AWQMarlinConfig(QuantizationConfig):
    def __init__(self, weight_bits: int, group_size: int, zero_point: bool,
                 modules_to_not_convert: Optional[List[str]] = None) -> None:
        if weight_bits != 4:
            raise ValueError(f"AWQ: only 4-bit weights are supported, got {weight_bits}")
        if group_size not in (-1, 32, 64, 128):
            raise ValueError(f"AWQ: unsupported group size {group_size}")
        self.weight_bits, self.group_size, self.zero_point = weight_bits, group_size, zero_point
        self.modules_to_not_convert = modules_to_not_convert or []

    def get_name(self) -> str:
        return "awq_marlin"

    @staticmethod
    def get_config_filenames() -> List[str]:
        return ["quant_config.json", "quantize_config.json"]

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "AWQMarlinConfig":
        bits = cls.get_from_keys(config, ["w_bit", "bits"])
        group = cls.get_from_keys(config, ["q_group_size", "group_size"])
        zp = bool(config.get("zero_point", True))
        return cls(int(bits), int(group), zp, config.get("modules_to_not_convert"))

    def get_quant_method(self, layer: Any, prefix: str = "") -> Optional[LinearMethodBase]:
        if any(m and m in prefix for m in self.modules_to_not_convert):
            return UnquantizedLinearMethod()
        return AWQLinearMethod(self.group_size, self.zero_point)


register_quantization("awq")(AWQMarlinConfig)

"""GPTQ / AutoGPTQ checkpoints (``quant_method: "gptq"``): 4-bit weights, group-wise scales, optional zero
points (the layout the reference repacks for Marlin in
``mllm-kernel/mllm_kernel/cuda/csrc/gemm/marlin/gptq_marlin_repack.cuh``).

Checkpoint tensors per linear: ``qweight`` int32 ``[K/8, N]`` (eight consecutive input channels per
word, low nibble first), ``qzeros`` int32 ``[K/g, N/8]`` (eight consecutive output channels per word;
the classic format stores ``zero - 1``), ``scales`` fp16 ``[K/g, N]`` and ``g_idx`` int32 ``[K]``;
``w[k, n] = (q[k, n] - zero[k // g, n]) * scale[k // g, n]``.  After loading the tensors are unpacked
once and laid out K-major like every other 4-bit scheme here — ``weight_packed`` int32 ``[N, K/8]``,
``weight_zeros`` uint8 ``[N, K/g]``, ``weight_scale`` ``[N, K/g]`` — and served by the tcgen05 W4A16
kernel.

``desc_act`` checkpoints (activation order: input channel ``k`` belongs to group ``g_idx[k]``, groups are
not contiguous) are served by sorting the input channels by group once at load — the weight rows are
permuted so that groups become contiguous again — and permuting the activation columns the same way before
every GEMM (the role of the reference's ``permute_cols`` kernel).  Not combined with an input-dimension
split across tensor-parallel ranks.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ... import ops
from ...layers.quantize_base import LinearMethodBase, UnquantizedLinearMethod, set_weight_attrs
from ..quant_config import QuantizationConfig, register_quantization
from .awq import pack_rows_natural


def unpack_words(packed: torch.Tensor, dim: int) -> torch.Tensor:
    """int32 words holding eight 4-bit values (low nibble first) -> uint8 values, expanded along ``dim``."""
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    nib = ((packed.unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8)          # [..., 8]
    if dim == 0:
        return nib.permute(0, 2, 1).reshape(packed.shape[0] * 8, packed.shape[1])
    return nib.reshape(packed.shape[0], packed.shape[1] * 8)


def pack_words(values: torch.Tensor, dim: int) -> torch.Tensor:
    """Inverse of :func:`unpack_words` (tests, checkpoint writers)."""
    v = values.to(torch.int64)
    v = v.reshape(-1, 8, v.shape[1]).permute(0, 2, 1) if dim == 0 else v.reshape(v.shape[0], -1, 8)
    word = torch.zeros(v.shape[:2], dtype=torch.int64, device=values.device)
    for i in range(8):
        word |= (v[..., i] & 0xF) << (4 * i)
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


class GPTQLinearMethod(LinearMethodBase):
    def __init__(self, group_size: int, sym: bool, zero_offset: int = 1, desc_act: bool = False) -> None:
        self.group_size, self.sym, self.zero_offset, self.desc_act = group_size, sym, zero_offset, desc_act

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra) -> None:
        n, k = sum(output_partition_sizes), input_size_per_partition
        g = k if self.group_size == -1 else self.group_size
        if n % 8 or k % 8 or k % g:
            raise ValueError(f"GPTQ: N={n} and K={k} must be divisible by 8, K by the group size {g}")
        if self.group_size == -1 and input_size != input_size_per_partition:
            raise ValueError("GPTQ: per-channel groups (group_size -1) cannot be split along the input dimension")
        if self.desc_act and input_size != input_size_per_partition:
            raise ValueError("GPTQ: activation-order checkpoints cannot be split along the input dimension "
                             "(row-parallel layers under tensor parallelism)")
        qweight = nn.Parameter(torch.zeros(k // 8, n, dtype=torch.int32), requires_grad=False)
        qzeros = nn.Parameter(torch.zeros(k // g, n // 8, dtype=torch.int32), requires_grad=False)
        scales = nn.Parameter(torch.zeros(k // g, n, dtype=params_dtype), requires_grad=False)
        g_idx = nn.Parameter(torch.zeros(k, dtype=torch.int32), requires_grad=False)
        set_weight_attrs(qweight, {"input_dim": 0, "output_dim": 1, "packed_dim": 0, "pack_factor": 8})
        set_weight_attrs(qzeros, {"input_dim": 0, "output_dim": 1, "packed_dim": 1, "pack_factor": 8})
        set_weight_attrs(scales, {"input_dim": 0, "output_dim": 1})
        set_weight_attrs(g_idx, {"input_dim": 0, "ignore_shard": True})   # the same for every fused output shard
        for p in (qweight, qzeros, scales, g_idx):
            set_weight_attrs(p, extra)
        layer.register_parameter("qweight", qweight)
        layer.register_parameter("qzeros", qzeros)
        layer.register_parameter("scales", scales)
        layer.register_parameter("g_idx", g_idx)
        layer.w4_group = g

    def process_weights_after_loading(self, layer) -> None:
        if not hasattr(layer, "qweight"):
            return
        q = unpack_words(layer.qweight.data, 0)                      # [K, N]
        z = unpack_words(layer.qzeros.data, 1)                       # [K/g, N]
        perm_buf = None
        g_idx = layer.g_idx.data.long()
        contiguous = torch.arange(g_idx.numel(), device=g_idx.device) // layer.w4_group
        if self.desc_act and not torch.equal(g_idx, contiguous):
            perm = torch.argsort(g_idx, stable=True)                 # input channels grouped by their scale group
            if not torch.equal(g_idx[perm], contiguous):
                raise ValueError("GPTQ: g_idx does not assign exactly group_size channels to every group")
            q = q[perm]
            perm_buf = perm.to(torch.int64)
        layer.register_buffer("act_perm", perm_buf, persistent=False)
        z = ((z.to(torch.int16) + self.zero_offset) & 0xF).to(torch.uint8)
        packed = pack_rows_natural(q.t().contiguous())               # [N, K/8]
        zeros = z.t().contiguous()                                   # [N, K/g]
        scale = layer.scales.data.t().contiguous()                   # [N, K/g]
        for name in ("qweight", "qzeros", "scales", "g_idx"):
            delattr(layer, name)
        layer.w4_interleaved = packed.is_cuda     # GPU: nibble order the GEMM kernel expands fastest
        if layer.w4_interleaved:
            packed = ops.w4a16_interleave(packed)
        layer.register_parameter("weight_packed", nn.Parameter(packed, requires_grad=False))
        layer.register_parameter("weight_zeros", nn.Parameter(zeros, requires_grad=False))
        layer.register_parameter("weight_scale", nn.Parameter(scale, requires_grad=False))

    def apply(self, layer, x, bias=None, residual=None):
        perm = getattr(layer, "act_perm", None)
        if perm is not None:
            x = x.index_select(-1, perm)
        y = ops.w4a16_gemm(x, layer.weight_packed, layer.weight_scale, layer.weight_zeros, layer.w4_group, bias,
                            interleaved=getattr(layer, "w4_interleaved", False))
        return y if residual is None else y + residual


@register_quantization("gptq")
class GPTQConfig(QuantizationConfig):
    def __init__(self, weight_bits: int, group_size: int, sym: bool, desc_act: bool, checkpoint_format: str = "gptq",
                 modules_to_not_convert: Optional[List[str]] = None) -> None:
        if weight_bits != 4:
            raise ValueError(f"GPTQ: only 4-bit weights are supported, got {weight_bits}")
        if group_size not in (-1, 32, 64, 128):
            raise ValueError(f"GPTQ: unsupported group size {group_size}")
        if desc_act and group_size == -1:
            desc_act = False      # one group: the order of the input channels does not matter
        self.weight_bits, self.group_size, self.sym, self.desc_act = weight_bits, group_size, sym, bool(desc_act)
        # "gptq_v2" files store the zero point itself, the classic format stores zero - 1
        self.zero_offset = 0 if checkpoint_format == "gptq_v2" else 1
        self.modules_to_not_convert = modules_to_not_convert or []

    def get_name(self) -> str:
        return "gptq"

    @staticmethod
    def get_config_filenames() -> List[str]:
        return ["quantize_config.json", "quant_config.json"]

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "GPTQConfig":
        return cls(int(cls.get_from_keys(config, ["bits", "w_bit"])), int(cls.get_from_keys(config, ["group_size", "q_group_size"])),
                   bool(config.get("sym", True)), bool(config.get("desc_act", False)),
                   str(config.get("checkpoint_format", "gptq")), config.get("modules_to_not_convert"))

    def get_quant_method(self, layer: Any, prefix: str = "") -> Optional[LinearMethodBase]:
        if any(m and m in prefix for m in self.modules_to_not_convert) or "lm_head" in prefix:
            return UnquantizedLinearMethod()
        return GPTQLinearMethod(self.group_size, self.sym, self.zero_offset, self.desc_act)


register_quantization("gptq_marlin")(GPTQConfig)

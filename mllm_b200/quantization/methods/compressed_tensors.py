"""compressed-tensors checkpoints (llm-compressor): W4A16 ``pack-quantized``, W8A8 ``int-quantized`` and W8A16
(expanded to 16 bits at load).

Config parsing, the ``ignore`` matching rules (exact prefix, path component, ``re:`` regex, with
``model.`` / ``model.language_model.`` prefixes stripped) and the checkpoint tensor contracts
follow pymllm/quantization/methods/compressed_tensors.py:135-246,249-468,504-641:

* W4A16: ``weight_packed`` int32 ``[N, K/8]`` (nibble i of word j = element 8j+i, stored with a
  bias of 8), ``weight_scale`` ``[N, K/g]``, ``weight_shape`` ``[2]``; symmetric, group size g.
* W8A8: ``weight`` int8 ``[N, K]``, ``weight_scale`` ``[N, 1]``; activations are quantised per
  token at run time (``scale = absmax / 127``).

The reference repacks into Marlin's ``mma.sync`` fragment order; here the packed rows are kept
K-major exactly as stored, because the tcgen05 kernels take the weight matrix as the K-major
128-row MMA operand and dequantise tiles in shared memory.
"""

from __future__ import annotations

import re
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ... import ops
from ...layers.quantize_base import LinearMethodBase, UnquantizedLinearMethod, set_weight_attrs
from ..quant_config import QuantizationConfig, register_quantization

SUPPORTED_GROUP_SIZES = (-1, 32, 64, 128)


class CompressedTensorsW4A16Method(LinearMethodBase):
    def __init__(self, group_size: int) -> None:
        if group_size not in SUPPORTED_GROUP_SIZES:
            raise ValueError(f"Unsupported compressed-tensors group_size: {group_size}")
        self.group_size = group_size

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra) -> None:
        n = sum(output_partition_sizes)
        k = input_size_per_partition
        g = k if self.group_size == -1 else self.group_size
        if k % 8 or k % g:
            raise ValueError(f"input size {k} must be divisible by 8 and by the group size {g}")
        if self.group_size != -1 and self.group_size < input_size and input_size_per_partition % self.group_size:
            raise ValueError("input_size_per_partition must be divisible by group_size")
        packed = nn.Parameter(torch.zeros(n, k // 8, dtype=torch.int32), requires_grad=False)
        set_weight_attrs(packed, {"input_dim": 1, "output_dim": 0, "packed_dim": 1, "pack_factor": 8})
        scale = nn.Parameter(torch.zeros(n, k // g, dtype=params_dtype), requires_grad=False)
        set_weight_attrs(scale, {"input_dim": 1, "output_dim": 0})
        shape = nn.Parameter(torch.zeros(2, dtype=torch.int64), requires_grad=False)
        set_weight_attrs(shape, {"ignore_shard": True})
        for p in (packed, scale, shape):
            set_weight_attrs(p, extra)
        layer.register_parameter("weight_packed", packed)
        layer.register_parameter("weight_scale", scale)
        layer.register_parameter("weight_shape", shape)
        layer.w4_group = g

    def process_weights_after_loading(self, layer) -> None:
        layer.weight_packed.data = layer.weight_packed.data.contiguous()
        if layer.weight_packed.is_cuda and not getattr(layer, "w4_interleaved", False):
            # GPU: nibble order the GEMM kernel expands fastest
            layer.weight_packed.data = ops.w4a16_interleave(layer.weight_packed.data)
            layer.w4_interleaved = True
        layer.weight_scale.data = layer.weight_scale.data.contiguous()
        # the fused projections were assembled shard by shard; record the true local shape
        layer.weight_shape.data = torch.tensor(
            [layer.weight_packed.shape[0], layer.weight_packed.shape[1] * 8], dtype=torch.int64,
            device=layer.weight_shape.device)

    def apply(self, layer, x, bias=None, residual=None):
        y = ops.w4a16_gemm(x, layer.weight_packed, layer.weight_scale, None, layer.w4_group, bias,
                           interleaved=getattr(layer, "w4_interleaved", False))
        return y if residual is None else y + residual


class CompressedTensorsW8A8Method(LinearMethodBase):
    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra) -> None:
        n = sum(output_partition_sizes)
        w = nn.Parameter(torch.zeros(n, input_size_per_partition, dtype=torch.int8), requires_grad=False)
        set_weight_attrs(w, {"input_dim": 1, "output_dim": 0})
        s = nn.Parameter(torch.zeros(n, 1, dtype=torch.float32), requires_grad=False)
        set_weight_attrs(s, {"output_dim": 0})
        for p in (w, s):
            set_weight_attrs(p, extra)
        layer.register_parameter("weight", w)
        layer.register_parameter("weight_scale", s)
        layer.out_dtype = params_dtype

    def process_weights_after_loading(self, layer) -> None:
        layer.weight.data = layer.weight.data.contiguous()
        layer.weight_scale = nn.Parameter(layer.weight_scale.data.reshape(-1).float().contiguous(),
                                          requires_grad=False)

    def apply(self, layer, x, bias=None, residual=None):
        x_q, x_s = ops.per_token_quant_int8(x)
        y = ops.int8_scaled_mm(x_q, layer.weight, x_s, layer.weight_scale, layer.out_dtype, bias)
        return y if residual is None else y + residual


class CompressedTensorsW8A16Method(UnquantizedLinearMethod):
    """8-bit symmetric weights (per channel or per group), 16-bit activations.  There is no 8-bit-weight GEMM
    here (the reference serves this scheme with Marlin): the weights are expanded to the serving dtype once,
    after loading, and the ordinary tcgen05 GEMM runs — same outputs as the dequantised model, no memory
    saving.  ``weight`` int8 ``[N, K]`` (``int-quantized``) or ``weight_packed`` int32 ``[N, K/4]``
    (``pack-quantized``: byte i of word j = element 4j+i, stored +128), ``weight_scale`` ``[N, K/g]``."""

    def __init__(self, group_size: int, packed: bool) -> None:
        self.group_size, self.packed = group_size, packed

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra) -> None:
        n, k = sum(output_partition_sizes), input_size_per_partition
        g = k if self.group_size in (-1, None) else self.group_size
        if k % g or (self.packed and k % 4):
            raise ValueError(f"W8A16: input size {k} must be divisible by the group size {g}")
        if self.packed:
            w = nn.Parameter(torch.zeros(n, k // 4, dtype=torch.int32), requires_grad=False)
            set_weight_attrs(w, {"input_dim": 1, "output_dim": 0, "packed_dim": 1, "pack_factor": 4})
            shape = nn.Parameter(torch.zeros(2, dtype=torch.int64), requires_grad=False)
            set_weight_attrs(shape, {"ignore_shard": True})
            set_weight_attrs(shape, extra)
            layer.register_parameter("weight_shape", shape)
        else:
            w = nn.Parameter(torch.zeros(n, k, dtype=torch.int8), requires_grad=False)
            set_weight_attrs(w, {"input_dim": 1, "output_dim": 0})
        sc = nn.Parameter(torch.zeros(n, k // g, dtype=params_dtype), requires_grad=False)
        set_weight_attrs(sc, {"input_dim": 1, "output_dim": 0})
        for p in (w, sc):
            set_weight_attrs(p, extra)
        layer.register_parameter("weight_packed" if self.packed else "weight", w)
        layer.register_parameter("weight_scale", sc)
        layer._w8_dtype, layer._w8_group = params_dtype, g

    def process_weights_after_loading(self, layer) -> None:
        if hasattr(layer, "weight_scale"):
            if self.packed:
                words = layer.weight_packed.data
                shifts = torch.arange(0, 32, 8, device=words.device, dtype=torch.int32)
                q = (((words.unsqueeze(-1) >> shifts) & 0xFF).to(torch.int16) - 128).reshape(words.shape[0], -1)
                delattr(layer, "weight_packed")
                if hasattr(layer, "weight_shape"):
                    delattr(layer, "weight_shape")
            else:
                q = layer.weight.data.to(torch.int16)
                delattr(layer, "weight")
            scale = layer.weight_scale.data.float().repeat_interleave(layer._w8_group, dim=1)
            delattr(layer, "weight_scale")
            w = nn.Parameter((q.float() * scale).to(layer._w8_dtype), requires_grad=False)
            set_weight_attrs(w, {"input_dim": 1, "output_dim": 0})
            layer.register_parameter("weight", w)
        super().process_weights_after_loading(layer)


def _signature(cfg: "CompressedTensorsConfig") -> str:
    """Which kernel family serves this config, or a clear error."""
    if cfg.weight_type not in (None, "int"):
        raise ValueError(f"compressed-tensors: unsupported weight type {cfg.weight_type!r}")
    if cfg.quant_format == "pack-quantized" and cfg.weight_bits == 4 and cfg.input_bits is None:
        if not cfg.symmetric:
            raise ValueError("compressed-tensors W4A16: only symmetric weights are supported")
        if cfg.actorder not in (None, "static", False):
            raise ValueError("compressed-tensors W4A16: activation reordering is not supported")
        return "w4a16"
    if cfg.weight_bits == 8 and cfg.input_bits is None and cfg.quant_format in ("int-quantized", "naive-quantized", "pack-quantized"):
        if not cfg.symmetric or cfg.weight_strategy not in ("channel", "group"):
            raise ValueError("compressed-tensors W8A16: weights must be symmetric, per channel or per group")
        return "w8a16"
    if cfg.quant_format in ("int-quantized", "naive-quantized") and cfg.weight_bits == 8 and cfg.input_bits == 8:
        if cfg.weight_strategy != "channel" or not cfg.symmetric:
            raise ValueError("compressed-tensors W8A8: weights must be per-channel symmetric")
        if cfg.input_strategy != "token" or not cfg.input_dynamic or not cfg.input_symmetric:
            raise ValueError("compressed-tensors W8A8: activations must be dynamic per-token symmetric")
        return "w8a8"
    raise ValueError(
        f"compressed-tensors: unsupported scheme format={cfg.quant_format!r} weight_bits={cfg.weight_bits} "
        f"input_bits={cfg.input_bits}")


@register_quantization("compressed-tensors")
class CompressedTensorsConfig(QuantizationConfig):
    def __init__(self, *, quant_format: str, ignore: List[str], weight_bits: int, group_size: Optional[int],
                 weight_strategy: Optional[str], weight_type: Optional[str], weight_dynamic: bool, symmetric: bool,
                 actorder: Optional[str], input_bits: Optional[int], input_strategy: Optional[str],
                 input_type: Optional[str], input_dynamic: bool, input_symmetric: bool) -> None:
        self.quant_format, self.ignore = quant_format, ignore
        self.weight_bits, self.group_size = weight_bits, group_size
        self.weight_strategy, self.weight_type = weight_strategy, weight_type
        self.weight_dynamic, self.symmetric, self.actorder = weight_dynamic, symmetric, actorder
        self.input_bits, self.input_strategy, self.input_type = input_bits, input_strategy, input_type
        self.input_dynamic, self.input_symmetric = input_dynamic, input_symmetric

    def get_name(self) -> str:
        return "compressed-tensors"

    @staticmethod
    def get_config_filenames() -> List[str]:
        return ["config.json"]

    @staticmethod
    def _normalize_ignore(entries: List[str]) -> List[str]:
        out = []
        for e in entries:
            if not e.startswith("re:"):
                for pre in ("model.language_model.", "model."):
                    if e.startswith(pre):
                        e = e[len(pre):]
                        break
            out.append(e)
        return out

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "CompressedTensorsConfig":
        group = config["config_groups"]["group_0"]
        w = group["weights"]
        a = group.get("input_activations") or {}
        has_a = bool(group.get("input_activations"))
        return cls(
            quant_format=config["format"], ignore=cls._normalize_ignore(list(config.get("ignore", []))),
            weight_bits=w["num_bits"], group_size=w.get("group_size"), weight_strategy=w.get("strategy"),
            weight_type=w.get("type"), weight_dynamic=bool(w.get("dynamic", False)), symmetric=w["symmetric"],
            actorder=w.get("actorder"), input_bits=a.get("num_bits") if has_a else None,
            input_strategy=a.get("strategy") if has_a else None, input_type=a.get("type") if has_a else None,
            input_dynamic=bool(a.get("dynamic", False)), input_symmetric=bool(a.get("symmetric", False)),
        )

    def is_ignored(self, prefix: str) -> bool:
        bare = prefix
        for pre in ("model.language_model.", "model."):
            if bare.startswith(pre):
                bare = bare[len(pre):]
                break
        dotted = f".{bare}."
        for ig in self.ignore:
            if not ig:
                continue
            if ig.startswith("re:"):
                if re.match(ig[3:], bare) or re.match(ig[3:], prefix):
                    return True
            elif bare.startswith(ig) or f".{ig}." in dotted:
                return True
        return False

    def get_quant_method(self, layer: Any, prefix: str = "") -> Optional[LinearMethodBase]:
        kind = _signature(self)
        if self.is_ignored(prefix):
            return UnquantizedLinearMethod()
        if kind == "w4a16":
            return CompressedTensorsW4A16Method(self.group_size if self.group_size is not None else -1)
        if kind == "w8a16":
            return CompressedTensorsW8A16Method(self.group_size if self.weight_strategy == "group" else -1,
                                                packed=self.quant_format == "pack-quantized")
        return CompressedTensorsW8A8Method()

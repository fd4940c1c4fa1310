"""FP8 (e4m3) weight checkpoints, e.g. the ``*-FP8`` releases with ``quant_method: "fp8"``.

Per linear the checkpoint holds ``weight`` in ``float8_e4m3fn`` ``[N, K]`` and either
``weight_scale_inv`` fp32 ``[ceil(N/bn), ceil(K/bk)]`` (one scale per ``weight_block_size`` block, usually
128 x 128) or a per-tensor ``weight_scale``; ``w = fp8 * scale``.  This build expands the weights to the
serving dtype once, after loading, and runs the ordinary 16-bit tcgen05 GEMM: the format is *accepted*
(same outputs as the dequantised model), it does not yet save memory or use the fp8 tensor-core path.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ...layers.quantize_base import LinearMethodBase, UnquantizedLinearMethod, set_weight_attrs
from ..quant_config import QuantizationConfig, register_quantization

FP8 = torch.float8_e4m3fn


class Fp8LinearMethod(UnquantizedLinearMethod):
    def __init__(self, block: Optional[List[int]]) -> None:
        self.block = list(block) if block else None

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **extra) -> None:
        n, k = sum(output_partition_sizes), input_size_per_partition
        w = nn.Parameter(torch.zeros(n, k, dtype=FP8), requires_grad=False)
        set_weight_attrs(w, {"input_dim": 1, "output_dim": 0})
        set_weight_attrs(w, extra)
        layer.register_parameter("weight", w)
        layer._fp8_dtype = params_dtype
        if self.block:
            bn, bk = self.block
            if any(s % bn for s in output_partition_sizes) or (k % bk and k != input_size):
                raise ValueError(f"fp8: partition sizes {output_partition_sizes} x {k} do not align with blocks {self.block}")
            s = nn.Parameter(torch.ones(n // bn, (k + bk - 1) // bk, dtype=torch.float32), requires_grad=False)
            set_weight_attrs(s, {"input_dim": 1, "output_dim": 0, "packed_dim": 0, "pack_factor": bn})
            set_weight_attrs(s, extra)
            layer.register_parameter("weight_scale_inv", s)
        else:
            s = nn.Parameter(torch.ones(len(output_partition_sizes), dtype=torch.float32), requires_grad=False)
            set_weight_attrs(s, {"per_tensor_scale": True, "sizes": list(output_partition_sizes)})
            s.weight_loader = self._load_tensor_scale
            layer.register_parameter("weight_scale", s)

    @staticmethod
    def _load_tensor_scale(param, loaded, shard_id=None) -> None:
        """One scalar per fused shard (q / k / v or gate / up each come with their own)."""
        idx = 0 if shard_id is None else ({"q": 0, "k": 1, "v": 2}.get(shard_id, shard_id))
        if shard_id is None and param.numel() > 1:
            param.data.fill_(float(loaded.reshape(-1)[0]))
        else:
            param.data[int(idx)] = float(loaded.reshape(-1)[0])

    def process_weights_after_loading(self, layer) -> None:
        w = layer.weight.data
        if w.dtype == FP8:
            wf = w.to(torch.float32)
            if hasattr(layer, "weight_scale_inv"):
                bn, bk = self.block
                s = layer.weight_scale_inv.data
                s = s.repeat_interleave(bn, 0)[: wf.shape[0]].repeat_interleave(bk, 1)[:, : wf.shape[1]]
                wf = wf * s
                delattr(layer, "weight_scale_inv")
            elif hasattr(layer, "weight_scale"):
                sizes = layer.weight_scale.sizes
                s = torch.cat([layer.weight_scale.data[i].expand(n) for i, n in enumerate(sizes)]).view(-1, 1)
                wf = wf * s
                delattr(layer, "weight_scale")
            attrs = {k: getattr(layer.weight, k) for k in ("input_dim", "output_dim", "weight_loader") if hasattr(layer.weight, k)}
            delattr(layer, "weight")
            p = nn.Parameter(wf.to(layer._fp8_dtype), requires_grad=False)
            set_weight_attrs(p, attrs)
            layer.register_parameter("weight", p)
        super().process_weights_after_loading(layer)


@register_quantization("fp8")
class Fp8Config(QuantizationConfig):
    def __init__(self, fmt: str = "e4m3", weight_block_size: Optional[List[int]] = None,
                 modules_to_not_convert: Optional[List[str]] = None) -> None:
        if fmt not in ("e4m3", "float8_e4m3fn"):
            raise ValueError(f"fp8: only e4m3 weights are supported, got {fmt!r}")
        self.weight_block_size = list(weight_block_size) if weight_block_size else None
        self.modules_to_not_convert = modules_to_not_convert or []

    def get_name(self) -> str:
        return "fp8"

    @staticmethod
    def get_config_filenames() -> List[str]:
        return []

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "Fp8Config":
        return cls(str(config.get("fmt", "e4m3")), config.get("weight_block_size"),
                   config.get("modules_to_not_convert") or config.get("ignored_layers"))

    def get_quant_method(self, layer: Any, prefix: str = "") -> Optional[LinearMethodBase]:
        if any(m and m in prefix for m in self.modules_to_not_convert) or "lm_head" in prefix:
            return UnquantizedLinearMethod()
        return Fp8LinearMethod(self.weight_block_size)

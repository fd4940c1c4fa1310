"""Quantised expert matrices of mixture-of-experts checkpoints.

The grouped expert GEMM runs on 16-bit weights.  A quantised MoE checkpoint (AWQ, GPTQ, compressed-tensors
W4A16 / W8A8 / W8A16, FP8) stores, per expert projection, the same tensors a quantised linear layer would; this
helper collects them as they stream in and, when a projection is complete, returns its dequantised ``[N, K]``
matrix, which the ordinary expert loader then places (and shards).  Attention and dense-MLP projections of the
same checkpoint keep their quantised kernels; only the experts are expanded."""

from __future__ import annotations

import re
from typing import Dict, Iterable, Optional, Tuple

import torch

# a tensor of one expert projection: "<...>.mlp.experts.<e>.<gate|up|down>_proj.<suffix>"
_QUANT_EXPERT_RE = re.compile(r"^(.*\.mlp\.experts\.\d+\.(?:gate_proj|up_proj|down_proj))\.(\w+)$")
_PLAIN = (torch.bfloat16, torch.float16, torch.float32)

_NEEDS = {
    "awq": ("qweight", "qzeros", "scales"),
    "gptq": ("qweight", "qzeros", "scales", "g_idx"),
    "ct_w4a16": ("weight_packed", "weight_scale", "weight_shape"),
    "ct_int8": ("weight", "weight_scale"),
    "fp8_block": ("weight", "weight_scale_inv"),
    "fp8_tensor": ("weight", "weight_scale"),
}


def _kind(quant_config) -> Optional[str]:
    name = quant_config.get_name() if quant_config is not None else None
    if name in ("awq", "awq_marlin"):
        return "awq"
    if name in ("gptq", "gptq_marlin"):
        if getattr(quant_config, "desc_act", False):
            raise NotImplementedError("activation-order GPTQ experts are not supported")
        return "gptq"
    if name == "compressed-tensors":
        return "ct_w4a16" if quant_config.weight_bits == 4 else "ct_int8"
    if name == "fp8":
        return "fp8_block" if quant_config.weight_block_size else "fp8_tensor"
    return None


class ExpertDequantizer:
    def __init__(self, quant_config, dtype: torch.dtype) -> None:
        self.cfg, self.kind, self.dtype = quant_config, _kind(quant_config), dtype
        self.pending: Dict[str, Dict[str, torch.Tensor]] = {}

    @property
    def active(self) -> bool:
        return self.kind is not None

    def suffixes(self):
        return _NEEDS[self.kind] if self.kind else ()

    def feed(self, projection: str, suffix: str, tensor) -> Optional[torch.Tensor]:
        """``projection``: name up to and excluding the tensor suffix.  Returns the ``[N, K]`` matrix once all
        tensors of the projection have arrived, else None."""
        t = tensor.materialize() if hasattr(tensor, "materialize") else tensor
        got = self.pending.setdefault(projection, {})
        got[suffix] = t
        if any(k not in got for k in _NEEDS[self.kind]):
            return None
        del self.pending[projection]
        return getattr(self, "_" + self.kind)(got).to(self.dtype)

    # ---- per format: everything in fp32, result [N, K] ----
    def _awq(self, t):
        from .methods.awq import unpack_awq

        q, z, s = unpack_awq(t["qweight"]).float(), unpack_awq(t["qzeros"]).float(), t["scales"].float()
        g = q.shape[0] // s.shape[0]
        return ((q - z.repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)).t()

    def _gptq(self, t):
        from .methods.gptq import unpack_words

        q, s = unpack_words(t["qweight"], 0).float(), t["scales"].float()
        z = ((unpack_words(t["qzeros"], 1).to(torch.int16) + self.cfg.zero_offset) & 0xF).float()
        g = q.shape[0] // s.shape[0]
        return ((q - z.repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)).t()

    def _ct_w4a16(self, t):
        from .methods.gptq import unpack_words

        q = unpack_words(t["weight_packed"], 1).float() - 8.0            # [N, K], offset-binary nibbles
        s = t["weight_scale"].float()
        return q * s.repeat_interleave(q.shape[1] // s.shape[1], 1)

    def _ct_int8(self, t):
        w, s = t["weight"].float(), t["weight_scale"].float().reshape(t["weight"].shape[0], -1)
        return w * s.repeat_interleave(w.shape[1] // s.shape[1], 1)

    def _fp8_block(self, t):
        w, s = t["weight"].float(), t["weight_scale_inv"].float()
        bn, bk = self.cfg.weight_block_size
        return w * s.repeat_interleave(bn, 0)[: w.shape[0]].repeat_interleave(bk, 1)[:, : w.shape[1]]

    def _fp8_tensor(self, t):
        return t["weight"].float() * float(t["weight_scale"].reshape(-1)[0])


def dequantized_experts(weights: Iterable[Tuple[str, torch.Tensor]], quant_config, dtype: torch.dtype):
    """Generator over ``(name, tensor)``: the tensors of every quantised expert projection are gathered and
    replaced by one dequantised ``<projection>.weight``; everything else, and experts the checkpoint left in
    16 / 32 bits, passes through unchanged."""
    dq = ExpertDequantizer(quant_config, dtype)
    if not dq.active:
        yield from weights
        return
    wanted = set(dq.suffixes())
    for name, tensor in weights:
        m = _QUANT_EXPERT_RE.match(name)
        plain = m is not None and m.group(2) == "weight" and tensor.dtype in _PLAIN
        if m is None or m.group(2) not in wanted or plain:
            yield name, tensor
            continue
        w = dq.feed(m.group(1), m.group(2), tensor)
        if w is not None:
            yield m.group(1) + ".weight", w
    if dq.pending:
        raise ValueError(f"incomplete quantised expert tensors for {sorted(dq.pending)[:3]} ...")

"""Write a seeded random-init checkpoint (HF layout: ``config.json`` + ``*.safetensors``).

Used to give benchmarks and tests a model directory without any download: matrices are
N(0, 0.02), norm gains are 1.  Tensors are written one decoder layer per shard so peak host
memory stays at one layer.  Covers the dense Qwen3 and Qwen3-MoE text models.
"""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, Optional

import torch

from ..models.presets import preset_to_config_json


def _randn(shape, gen, device, dtype, std):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype).cpu()


def write_random_checkpoint(preset: str, out_dir, seed: int = 0, std: float = 0.02,
                            dtype: torch.dtype = torch.bfloat16, device: Optional[str] = None,
                            tp_shard: int = 1) -> Path:
    """``tp_shard = N > 1`` writes the checkpoint of ONE tensor-parallel rank of an N-way split of the dense
    model, for runners that have no sharded loading of their own: ``config.json`` names the per-rank head
    counts and intermediate size, q / k / v / gate / up have per-rank shapes, and o_proj / down_proj keep
    their full input width so that a row-parallel layer can cut out its own slice."""
    from safetensors.torch import save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    cfg = preset_to_config_json(preset)
    full_q = full_inter = None
    if tp_shard > 1:
        tcfg = cfg.get("text_config", cfg)
        if tcfg.get("num_experts", 0):
            raise ValueError("tp_shard is for dense models")
        if tcfg["num_attention_heads"] % tp_shard or tcfg["intermediate_size"] % tp_shard:
            raise ValueError(f"heads / intermediate size not divisible by {tp_shard}")
        full_q = tcfg["num_attention_heads"] * tcfg["head_dim"]
        full_inter = tcfg["intermediate_size"]
        tcfg["num_attention_heads"] //= tp_shard
        tcfg["num_key_value_heads"] = max(1, tcfg["num_key_value_heads"] // tp_shard)
        tcfg["intermediate_size"] //= tp_shard
    done_marker = out / ".complete"
    if done_marker.exists():
        return out
    with open(out / "config.json", "w") as f:
        json.dump(cfg, f, indent=1)
    tc = cfg.get("text_config", cfg)
    H, L = tc["hidden_size"], tc["num_hidden_layers"]
    hq, hkv, D = tc["num_attention_heads"], tc["num_key_value_heads"], tc["head_dim"]
    inter, V = tc["intermediate_size"], tc["vocab_size"]
    n_exp = tc.get("num_experts", 0)
    moe_inter = tc.get("moe_intermediate_size", 0)
    dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    index: Dict[str, str] = {}

    def dump(name: str, tensors: Dict[str, torch.Tensor]) -> None:
        save_file(tensors, str(out / name))
        for k in tensors:
            index[k] = name

    head = {"model.embed_tokens.weight": _randn((V, H), gen, dev, dtype, std),
            "model.norm.weight": torch.ones(H, dtype=dtype)}
    if not tc.get("tie_word_embeddings", False):
        head["lm_head.weight"] = _randn((V, H), gen, dev, dtype, std)
    dump("model-embed.safetensors", head)
    for i in range(L):
        p = f"model.layers.{i}."
        t = {
            p + "self_attn.q_proj.weight": _randn((hq * D, H), gen, dev, dtype, std),
            p + "self_attn.k_proj.weight": _randn((hkv * D, H), gen, dev, dtype, std),
            p + "self_attn.v_proj.weight": _randn((hkv * D, H), gen, dev, dtype, std),
            p + "self_attn.o_proj.weight": _randn((H, full_q or hq * D), gen, dev, dtype, std),
            p + "self_attn.q_norm.weight": torch.ones(D, dtype=dtype),
            p + "self_attn.k_norm.weight": torch.ones(D, dtype=dtype),
            p + "input_layernorm.weight": torch.ones(H, dtype=dtype),
            p + "post_attention_layernorm.weight": torch.ones(H, dtype=dtype),
        }
        if n_exp:
            t[p + "mlp.gate.weight"] = _randn((n_exp, H), gen, dev, dtype, std)
            for e in range(n_exp):
                t[p + f"mlp.experts.{e}.gate_proj.weight"] = _randn((moe_inter, H), gen, dev, dtype, std)
                t[p + f"mlp.experts.{e}.up_proj.weight"] = _randn((moe_inter, H), gen, dev, dtype, std)
                t[p + f"mlp.experts.{e}.down_proj.weight"] = _randn((H, moe_inter), gen, dev, dtype, std)
        else:
            t[p + "mlp.gate_proj.weight"] = _randn((inter, H), gen, dev, dtype, std)
            t[p + "mlp.up_proj.weight"] = _randn((inter, H), gen, dev, dtype, std)
            t[p + "mlp.down_proj.weight"] = _randn((H, full_inter or inter), gen, dev, dtype, std)
        dump(f"model-layer-{i:03d}.safetensors", t)
    with open(out / "model.safetensors.index.json", "w") as f:
        json.dump({"metadata": {}, "weight_map": index}, f)
    done_marker.write_text("ok")
    return out

"""Built-in model shapes so benchmarks and tests can run without a checkpoint directory.

Each preset is a plain attribute bag with the HF ``config.json`` field names the
models read.  Shapes: Qwen3 dense (0.6B / 1.7B / 4B / 8B / 14B / 32B), Qwen3-30B-A3B
(MoE), Llama / Qwen2 decoders, the Qwen3.5 hybrids, and the vision+language pairs Qwen3-VL-2B, Qwen2-VL-2B
and Qwen2.5-VL-3B (each with a ``-tiny`` shape for tests).
"""

from __future__ import annotations

import copy
from types import SimpleNamespace
from typing import Any, Dict


def _dense(hidden, layers, heads, kv, inter, tie, vocab=151936, theta=1e6) -> Dict[str, Any]:
    return dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=hidden, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=kv, head_dim=128, intermediate_size=inter,
        vocab_size=vocab, rms_norm_eps=1e-6, rope_theta=theta, tie_word_embeddings=tie,
        max_position_embeddings=40960, attention_bias=False, hidden_act="silu", torch_dtype="bfloat16",
        eos_token_id=151645, bos_token_id=151643,
    )


PRESETS: Dict[str, Dict[str, Any]] = {
    "qwen3-0.6b": _dense(1024, 28, 16, 8, 3072, True),
    "qwen3-1.7b": _dense(2048, 28, 16, 8, 6144, True),
    "qwen3-4b": _dense(2560, 36, 32, 8, 9728, True),
    "qwen3-8b": _dense(4096, 36, 32, 8, 12288, False),
    "qwen3-14b": _dense(5120, 40, 40, 8, 17408, False),
    "qwen3-32b": _dense(5120, 64, 64, 8, 25600, False),
    "qwen3-tiny": _dense(256, 2, 4, 2, 512, True, vocab=1024),
}
PRESETS["qwen3-30b-a3b"] = dict(
    _dense(2048, 48, 32, 4, 6144, False),
    architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", num_experts=128, num_experts_per_tok=8,
    moe_intermediate_size=768, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
)
PRESETS["qwen3-moe-tiny"] = dict(
    _dense(256, 2, 4, 2, 512, True, vocab=1024),
    architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", num_experts=8, num_experts_per_tok=2,
    moe_intermediate_size=256, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
)
# Llama / Qwen2 families (same decoder stack without q/k norms; published shapes)
PRESETS["llama-3.1-8b"] = dict(
    _dense(4096, 32, 32, 8, 14336, False, vocab=128256, theta=5e5),
    architectures=["LlamaForCausalLM"], model_type="llama", rms_norm_eps=1e-5, max_position_embeddings=131072,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192), eos_token_id=128009, bos_token_id=128000,
)
PRESETS["qwen2.5-7b"] = dict(
    _dense(3584, 28, 28, 4, 18944, False, vocab=152064, theta=1e6),
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", max_position_embeddings=32768,
)
PRESETS["llama-tiny"] = dict(_dense(256, 2, 4, 2, 512, True, vocab=1024, theta=1e4),
                             architectures=["LlamaForCausalLM"], model_type="llama")
PRESETS["qwen2-tiny"] = dict(_dense(256, 2, 4, 2, 512, True, vocab=1024), architectures=["Qwen2ForCausalLM"], model_type="qwen2")


def _hybrid(hidden, layers, heads, kv_heads, inter, head_dim, lin_k_heads, lin_v_heads, vocab=151936):
    return dict(
        architectures=["Qwen3_5ForCausalLM"], model_type="qwen3_5_text", vocab_size=vocab, hidden_size=hidden,
        intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads,
        head_dim=head_dim, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=32768, attention_bias=False,
        hidden_act="silu", linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_value_head_dim=128,
        linear_num_key_heads=lin_k_heads, linear_num_value_heads=lin_v_heads, full_attention_interval=4,
        layer_types=["full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(layers)],
        rope_parameters=dict(rope_theta=1e7, partial_rotary_factor=0.25, rope_type="default", mrope_section=[11, 11, 10]),
        torch_dtype="bfloat16", eos_token_id=151645,
    )


PRESETS["qwen3.5-2b"] = _hybrid(2048, 24, 8, 2, 6144, 256, 16, 16)
PRESETS["qwen3.5-tiny"] = dict(_hybrid(256, 4, 2, 1, 512, 128, 1, 2, vocab=1024),
                               rope_parameters=dict(rope_theta=1e4, partial_rotary_factor=0.25, rope_type="default",
                                                    mrope_section=[6, 5, 5]))
_VL_VISION = dict(
    depth=24, hidden_size=1024, num_heads=16, intermediate_size=4096, patch_size=16, temporal_patch_size=2,
    spatial_merge_size=2, in_channels=3, out_hidden_size=2048, num_position_embeddings=2304,
    deepstack_visual_indexes=[5, 11, 17], hidden_act="gelu_pytorch_tanh",
)
PRESETS["qwen3-vl-2b"] = dict(
    architectures=["Qwen3VLForConditionalGeneration"], model_type="qwen3_vl", tie_word_embeddings=True,
    image_token_id=151655, video_token_id=151656, vision_start_token_id=151652, vision_end_token_id=151653,
    text_config=dict(_dense(2048, 28, 16, 8, 6144, True, theta=5e6),
                     rope_scaling=dict(mrope_section=[24, 20, 20], mrope_interleaved=True, rope_type="default")),
    vision_config=_VL_VISION, torch_dtype="bfloat16", eos_token_id=151645,
)
PRESETS["qwen3-vl-tiny"] = dict(
    architectures=["Qwen3VLForConditionalGeneration"], model_type="qwen3_vl", tie_word_embeddings=True,
    image_token_id=1001, video_token_id=1002, vision_start_token_id=1003, vision_end_token_id=1004,
    text_config=dict(_dense(256, 3, 2, 1, 512, True, vocab=1024, theta=5e6),
                     rope_scaling=dict(mrope_section=[24, 20, 20], mrope_interleaved=True, rope_type="default")),
    vision_config=dict(depth=3, hidden_size=128, num_heads=2, intermediate_size=256, patch_size=16,
                       temporal_patch_size=2, spatial_merge_size=2, in_channels=3, out_hidden_size=256,
                       num_position_embeddings=64, deepstack_visual_indexes=[0, 1],
                       hidden_act="gelu_pytorch_tanh"),
    torch_dtype="bfloat16", eos_token_id=1,
)

# Qwen2-VL / Qwen2.5-VL: Qwen2 decoder (biased q / k / v, sectioned 3-D rope) behind their own vision towers
_Q2VL_IDS = dict(image_token_id=151655, video_token_id=151656, vision_start_token_id=151652, vision_end_token_id=151653)
_Q2VL_TINY_IDS = dict(image_token_id=1001, video_token_id=1002, vision_start_token_id=1003, vision_end_token_id=1004)


def _qwen2_text(hidden, layers, heads, kv, inter, tie, vocab=151936, sections=(16, 24, 24)) -> Dict[str, Any]:
    d = _dense(hidden, layers, heads, kv, inter, tie, vocab=vocab, theta=1e6)
    d.update(architectures=["Qwen2ForCausalLM"], model_type="qwen2", head_dim=hidden // heads, max_position_embeddings=32768,
             rope_scaling=dict(type="mrope", mrope_section=list(sections)))
    return d


PRESETS["qwen2-vl-2b"] = dict(
    architectures=["Qwen2VLForConditionalGeneration"], model_type="qwen2_vl", tie_word_embeddings=True, **_Q2VL_IDS,
    text_config=_qwen2_text(1536, 28, 12, 2, 8960, True),
    vision_config=dict(depth=32, embed_dim=1280, hidden_size=1536, num_heads=16, mlp_ratio=4, patch_size=14,
                       spatial_merge_size=2, temporal_patch_size=2, in_channels=3, hidden_act="quick_gelu"),
    torch_dtype="bfloat16", eos_token_id=151645,
)
PRESETS["qwen2-vl-tiny"] = dict(
    architectures=["Qwen2VLForConditionalGeneration"], model_type="qwen2_vl", tie_word_embeddings=True, **_Q2VL_TINY_IDS,
    text_config=_qwen2_text(256, 2, 4, 2, 512, True, vocab=1024, sections=(8, 12, 12)),
    vision_config=dict(depth=2, embed_dim=64, hidden_size=256, num_heads=2, mlp_ratio=2, patch_size=14,
                       spatial_merge_size=2, temporal_patch_size=2, in_channels=3, hidden_act="quick_gelu"),
    torch_dtype="bfloat16", eos_token_id=1,
)
PRESETS["qwen2.5-vl-3b"] = dict(
    architectures=["Qwen2_5_VLForConditionalGeneration"], model_type="qwen2_5_vl", tie_word_embeddings=True, **_Q2VL_IDS,
    text_config=_qwen2_text(2048, 36, 16, 2, 11008, True),
    vision_config=dict(depth=32, hidden_size=1280, hidden_act="silu", intermediate_size=3420, num_heads=16, in_channels=3,
                       patch_size=14, spatial_merge_size=2, temporal_patch_size=2, window_size=112, out_hidden_size=2048,
                       fullatt_block_indexes=[7, 15, 23, 31], tokens_per_second=2),
    torch_dtype="bfloat16", eos_token_id=151645,
)
PRESETS["qwen2.5-vl-tiny"] = dict(
    architectures=["Qwen2_5_VLForConditionalGeneration"], model_type="qwen2_5_vl", tie_word_embeddings=True, **_Q2VL_TINY_IDS,
    text_config=_qwen2_text(256, 2, 4, 2, 512, True, vocab=1024, sections=(8, 12, 12)),
    vision_config=dict(depth=3, hidden_size=64, hidden_act="silu", intermediate_size=96, num_heads=2, in_channels=3,
                       patch_size=14, spatial_merge_size=2, temporal_patch_size=2, window_size=56, out_hidden_size=256,
                       fullatt_block_indexes=[1], tokens_per_second=2),
    torch_dtype="bfloat16", eos_token_id=1,
)


def _to_ns(d: Dict[str, Any]) -> SimpleNamespace:
    ns = SimpleNamespace()
    for k, v in d.items():
        setattr(ns, k, _to_ns(v) if isinstance(v, dict) and k.endswith("_config") else copy.deepcopy(v))
    return ns


def get_preset(name: str, **overrides) -> SimpleNamespace:
    key = name.lower()
    if key not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; have {sorted(PRESETS)}")
    d = copy.deepcopy(PRESETS[key])
    d.update(overrides)
    return _to_ns(d)


def preset_to_config_json(name: str) -> Dict[str, Any]:
    """The preset as a HF-style ``config.json`` dict (used to materialise random checkpoints)."""
    return copy.deepcopy(PRESETS[name.lower()])

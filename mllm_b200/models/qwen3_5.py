"""Qwen3.5 hybrid decoder (Qwen3_5ForCausalLM): gated-delta-net layers interleaved with gated full
attention (roles of pymllm/models/qwen3_5.py:71-1087; math checked against HF ``modeling_qwen3_5``).

Per layer: ``x += mixer(norm(x)); x += mlp(norm(x))`` with zero-centred RMSNorm gains (``1 + w``, folded
into the stored weight at load).  The mixer is :class:`GatedDeltaNet` or full attention with per-head
q/k norm, partial rotary embedding on the first ``head_dim * partial_rotary_factor`` features (interleaved
M-RoPE axes when 3-D positions are given), KV cache, and an output gate ``attn * sigmoid(gate)`` whose
gate comes from the doubled q projection.

Status of the device path: the GEMMs, norms, SwiGLU MLP, KV write, conv / recurrent-state kernels and
(for head_dim 128) attention run on the sm_100a kernels; head_dim 256 attention (the published Qwen3.5
shape) falls back to the PyTorch statement of attention, and the layers are not tensor-parallel yet.
"""

from __future__ import annotations

import time
from typing import Iterable, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..engine.forward_batch import ForwardBatch
from ..layers import MLP, GemmaRMSNorm, VocabParallelEmbedding
from ..layers.gdn import GatedDeltaNet
from ..mem_cache import GDNPool
from ..ops import reference as ref
from ..parallel import state as pstate
from .qwen3 import LogitsProcessorOutput
from .qwen3_vl import VisionLanguageMixin


def _rope_params(config) -> dict:
    rp = getattr(config, "rope_parameters", None) or getattr(config, "rope_scaling", None) or {}
    return rp if isinstance(rp, dict) else vars(rp)


class Qwen3_5Attention(nn.Module):
    def __init__(self, config, layer_id: int, params_dtype=None) -> None:
        super().__init__()
        dt = params_dtype or torch.get_default_dtype()
        self.layer_id = layer_id
        # tensor parallelism: query heads are split over the ranks; KV heads too, or replicated when there
        # are fewer of them than ranks; the output projection is row-parallel (all-reduce of partial sums)
        self.tp, self.tp_rank = pstate.get_tensor_model_parallel_world_size(), pstate.get_tensor_model_parallel_rank()
        hq, hkv = config.num_attention_heads, config.num_key_value_heads
        if hq % self.tp or (hkv % self.tp and self.tp % hkv):
            raise ValueError(f"attention: {hq} query / {hkv} KV heads do not divide over {self.tp} ranks")
        self.total_heads, self.total_kv_heads = hq, hkv
        self.num_heads, self.num_kv_heads = hq // self.tp, max(1, hkv // self.tp)
        self.kv_head_start = (self.tp_rank * hkv) // self.tp
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        H = config.hidden_size
        rp = _rope_params(config)
        self.theta = float(rp.get("rope_theta", getattr(config, "rope_theta", 1e4)))
        self.rotary_dim = int(self.head_dim * float(rp.get("partial_rotary_factor", getattr(config, "partial_rotary_factor", 1.0))))
        self.mrope_section = rp.get("mrope_section", [11, 11, 10])
        eps = getattr(config, "rms_norm_eps", 1e-6)
        D = self.head_dim

        def lin(o, i, loader):
            m = nn.Module()
            m.weight = nn.Parameter(torch.empty(o, i, dtype=dt), requires_grad=False)
            m.weight.weight_loader = loader
            return m

        def rows(start, count):
            return lambda p, full, shard_id=None: p.data.copy_(full[start:start + count])

        self.q_proj = lin(self.num_heads * D * 2, H, rows(self.tp_rank * self.num_heads * 2 * D, self.num_heads * 2 * D))  # per head: [query(D) | gate(D)]
        self.k_proj = lin(self.num_kv_heads * D, H, rows(self.kv_head_start * D, self.num_kv_heads * D))
        self.v_proj = lin(self.num_kv_heads * D, H, rows(self.kv_head_start * D, self.num_kv_heads * D))
        c0, cn = self.tp_rank * self.num_heads * D, self.num_heads * D
        self.o_proj = lin(H, self.num_heads * D, lambda p, full, shard_id=None: p.data.copy_(full[:, c0:c0 + cn]))
        self.q_norm = GemmaRMSNorm(self.head_dim, eps, dt)
        self.k_norm = GemmaRMSNorm(self.head_dim, eps, dt)
        self.scale = self.head_dim ** -0.5

    def _cos_sin(self, fb: ForwardBatch):
        half = self.rotary_dim // 2
        inv = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, device=fb.positions.device, dtype=torch.float32) / self.rotary_dim))
        if fb.mrope_positions is not None:
            ang = fb.mrope_positions.float().unsqueeze(-1) * inv           # [3, T, half]
            out = ang[0].clone()
            for axis, offset in ((1, 1), (2, 2)):                           # interleaved t/h/w layout
                n = min(self.mrope_section[axis] * 3, half)
                idx = torch.arange(offset, n, 3, device=out.device)
                out[:, idx] = ang[axis][:, idx]
            ang = out
        else:
            ang = fb.positions.float().unsqueeze(-1) * inv
        return ang.cos(), ang.sin()

    def forward(self, x: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        T, D = x.shape[0], self.head_dim
        qg = ops.linear(x, self.q_proj.weight).view(T, self.num_heads, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(T, self.num_heads * D)
        k = ops.linear(x, self.k_proj.weight).view(T, self.num_kv_heads, D)
        v = ops.linear(x, self.v_proj.weight).view(T, self.num_kv_heads, D)
        q = self.q_norm(q.reshape(-1, D)).view(T, self.num_heads, D)
        k = self.k_norm(k.reshape(-1, D)).view(T, self.num_kv_heads, D)
        cos, sin = self._cos_sin(fb)
        q = ref.apply_rope_neox(q.float(), cos, sin).to(x.dtype).contiguous()
        k = ref.apply_rope_neox(k.float(), cos, sin).to(x.dtype).contiguous()
        kc, vc = fb.token_to_kv_pool.get_kv_buffer(self.layer_id)
        ops.kv_write(k.reshape(T, -1), v.reshape(T, -1), fb.out_cache_loc, kc, vc)
        rtt = fb.req_to_token_pool.req_to_token
        # head sizes 64 / 128 / 256 run on the attention kernels; ops falls back to library / PyTorch paths otherwise
        if fb.forward_mode.is_decode():
            o = ops.attention_decode(q, kc, vc, rtt, fb.req_pool_indices, fb.seq_lens, self.scale, max_seq_len=fb.max_seq_len)
        else:
            ext_cpu, pre_cpu = getattr(fb, "extend_seq_lens_cpu", None), getattr(fb, "extend_prefix_lens_cpu", None)
            seq_cpu = [a + b for a, b in zip(ext_cpu, pre_cpu)] if ext_cpu is not None and pre_cpu is not None else None
            o = ops.attention_prefill(q, kc, vc, rtt, fb.req_pool_indices, fb.seq_lens, fb.extend_prefix_lens,
                                      fb.extend_start_loc, self.scale, max_q_len=fb.max_extend_len,
                                      seq_lens_cpu=seq_cpu, prefix_lens_cpu=pre_cpu)
        o = o.reshape(T, self.num_heads * D) * torch.sigmoid(gate.float()).to(x.dtype)
        y = ops.linear(o, self.o_proj.weight)
        return pstate.tensor_model_parallel_all_reduce(y) if self.tp > 1 else y


class Qwen3_5DecoderLayer(nn.Module):
    def __init__(self, config, layer_id: int, attn_index: int, gdn_index: int, quant_config=None, params_dtype=None) -> None:
        super().__init__()
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.layer_type = config.layer_types[layer_id]
        if self.layer_type == "linear_attention":
            self.linear_attn = GatedDeltaNet(config, layer_id, gdn_index, params_dtype)
        else:
            self.self_attn = Qwen3_5Attention(config, attn_index, params_dtype)
        self.mlp = self._make_mlp(config, layer_id, quant_config, params_dtype)
        self.input_layernorm = GemmaRMSNorm(config.hidden_size, eps, params_dtype)
        self.post_attention_layernorm = GemmaRMSNorm(config.hidden_size, eps, params_dtype)

    def _make_mlp(self, config, layer_id, quant_config, params_dtype):
        return MLP(config.hidden_size, config.intermediate_size, quant_config, f"model.layers.{layer_id}.mlp",
                   params_dtype, reduce_results=True)

    def forward(self, hidden, residual, fb):
        if residual is None:
            residual = hidden
            hidden = self.input_layernorm(hidden)
        else:
            hidden, residual = self.input_layernorm(hidden, residual)
        hidden = self.linear_attn(hidden, fb) if self.layer_type == "linear_attention" else self.self_attn(hidden, fb)
        hidden, residual = self.post_attention_layernorm(hidden, residual)
        return self.mlp(hidden), residual


class Qwen3_5Model(nn.Module):
    layer_cls = Qwen3_5DecoderLayer

    def __init__(self, config, quant_config=None, params_dtype=None) -> None:
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, params_dtype, shard=False)
        layers, a, g = [], 0, 0
        for i in range(config.num_hidden_layers):
            layers.append(self.layer_cls(config, i, a, g, quant_config, params_dtype))
            if config.layer_types[i] == "linear_attention":
                g += 1
            else:
                a += 1
        self.layers = nn.ModuleList(layers)
        self.num_attn_layers, self.num_gdn_layers = a, g
        self.norm = GemmaRMSNorm(config.hidden_size, getattr(config, "rms_norm_eps", 1e-6), params_dtype)

    def forward(self, input_ids, fb, input_embeds=None):
        hidden = self.embed_tokens(input_ids) if input_embeds is None else input_embeds
        residual = None
        for layer in self.layers:
            hidden, residual = layer(hidden, residual, fb)
        hidden, _ = self.norm(hidden, residual)
        return hidden


class Qwen3_5ForCausalLM(nn.Module):
    """Text model.  ``kv_layers`` tells the runner to size the KV pool for the full-attention layers only;
    the gated-delta-net state pool is created on first use, one row per request slot."""

    model_cls = Qwen3_5Model

    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None) -> None:
        super().__init__()
        config = getattr(config, "text_config", config)
        if not getattr(config, "layer_types", None):
            interval = getattr(config, "full_attention_interval", 4)
            config.layer_types = ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
                                  for i in range(config.num_hidden_layers)]
        self.config = config
        self.quant_config = quant_config
        self.model = self.model_cls(config, quant_config, params_dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        if not self.tie:
            self.lm_head = VocabParallelEmbedding(config.vocab_size, config.hidden_size, params_dtype, shard=False)
        self.kv_layers = self.model.num_attn_layers
        self._gdn_pool: Optional[GDNPool] = None

    def make_gdn_pool(self, slots: int, track_slots: int = 0) -> GDNPool:
        """State rows for ``slots`` requests plus ``track_slots`` snapshot rows for the prefix cache
        (this rank's heads only under tensor parallelism)."""
        c = self.config
        w = self.model.embed_tokens.weight
        gdn = next(m for m in self.modules() if isinstance(m, GatedDeltaNet))
        self._gdn_pool = GDNPool(self.model.num_gdn_layers, slots, gdn.num_v_heads, c.linear_key_head_dim,
                                 c.linear_value_head_dim, gdn.conv_dim, c.linear_conv_kernel_dim, w.device, w.dtype,
                                 track_slots=track_slots)
        return self._gdn_pool

    def gdn_pool(self, fb: ForwardBatch) -> GDNPool:
        slots = fb.req_to_token_pool.req_to_token.shape[0]
        if self._gdn_pool is None or self._gdn_pool.slots != slots:
            self.make_gdn_pool(slots)
        return self._gdn_pool

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.model.embed_tokens.weight if self.tie else self.lm_head.weight

    def forward(self, input_ids, positions, forward_batch: ForwardBatch, input_embeds=None) -> LogitsProcessorOutput:
        fb = forward_batch
        fb.extra["gdn_pool"] = self.gdn_pool(fb)
        t0 = time.perf_counter()
        hidden = self.model(input_ids, fb, input_embeds)
        if fb.forward_mode.is_extend() and fb.extend_seq_lens is not None:
            hidden = hidden.index_select(0, torch.cumsum(fb.extend_seq_lens, 0) - 1)
        logits = ops.linear(hidden, self.lm_head_weight)
        ms = (time.perf_counter() - t0) * 1e3
        if fb.forward_mode.is_decode():
            fb.llm_decode_ms = ms
        else:
            fb.llm_prefill_ms = ms
        return LogitsProcessorOutput(next_token_logits=logits[:, : self.config.vocab_size])

    # ------------------------------------------------------------------ loading
    _OFFSET_NORMS = ("input_layernorm.weight", "post_attention_layernorm.weight", "q_norm.weight", "k_norm.weight")

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        params = dict(self.named_parameters())
        loaded = set()
        for name, t in weights:
            for old, new in (("model.language_model.", "model."), ("language_model.model.", "model."), ("language_model.", "model.")):
                if name.startswith(old):
                    name = new + name[len(old):]
                    break
            if name.startswith(("visual.", "model.visual.", "mtp.")) or "rotary_emb.inv_freq" in name:
                continue
            if name.startswith("lm_head.") and self.tie:
                continue
            target = name
            if (".gate_proj." in name or ".up_proj." in name) and ".experts." not in name:
                is_gate = ".gate_proj." in name
                target = name.replace(".gate_proj.", ".gate_up_proj.") if is_gate else name.replace(".up_proj.", ".gate_up_proj.")
                p = params.get(target)
                if p is None:
                    continue
                p.weight_loader(p, t, 0 if is_gate else 1)
                loaded.add(target + (":gate" if is_gate else ":up"))
                continue
            p = params.get(target)
            if p is None:
                continue
            if name.endswith(self._OFFSET_NORMS) or name == "model.norm.weight":
                p.data.copy_((t.float() + 1.0).to(p.dtype))          # zero-centred gain: store 1 + w
            elif hasattr(p, "weight_loader"):
                p.weight_loader(p, t)                                 # sharded / reshaped by the layer
            else:
                p.data.copy_(t.reshape(p.shape))
            loaded.add(target)
        # both halves of every fused gate/up weight must have arrived
        halves = {n.rsplit(':', 1)[0] for n in loaded if n.endswith((':gate', ':up'))}
        for h in halves:
            if h + ':gate' in loaded and h + ':up' in loaded:
                loaded.add(h)
        return {n for n in loaded if not n.endswith((':gate', ':up'))}

    def post_load(self) -> None:
        for m in self.modules():
            if isinstance(m, GatedDeltaNet):
                m.fuse_small_projections()


class Qwen3_5ForConditionalGeneration(VisionLanguageMixin, Qwen3_5ForCausalLM):
    """Vision-language variant: the Qwen3-VL style vision tower (no deepstack taps) in front of the hybrid
    text model; image features replace the image-token rows of the input embeddings and the full-attention
    layers rotate with 3-D (t, h, w) positions.  A checkpoint of this layout without a ``vision_config``
    is served as text only (its vision tensors, if any, are skipped)."""

    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None) -> None:
        tc = getattr(config, "text_config", config)
        if not hasattr(tc, "tie_word_embeddings"):
            tc.tie_word_embeddings = bool(getattr(config, "tie_word_embeddings", False))
        Qwen3_5ForCausalLM.__init__(self, config, quant_config, params_dtype)
        self.hidden_size = tc.hidden_size
        self.has_vision = getattr(config, "vision_config", None) is not None and getattr(config, "image_token_id", None) is not None
        if self.has_vision:
            self._init_vision(config, params_dtype or torch.get_default_dtype())
        self.uses_mrope = self.has_vision

    def forward(self, input_ids, positions, forward_batch: ForwardBatch, input_embeds=None) -> LogitsProcessorOutput:
        fb = forward_batch
        if self.has_vision:
            self._set_mrope_positions(input_ids, fb)
            embeds, _ = self._vision_embeds(input_ids, fb)
            if embeds is not None:
                input_embeds = embeds
        return Qwen3_5ForCausalLM.forward(self, input_ids, positions, fb, input_embeds)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        if not self.has_vision:
            return Qwen3_5ForCausalLM.load_weights(self, weights)
        loaded, rest = self._load_visual(weights)
        return loaded | Qwen3_5ForCausalLM.load_weights(self, rest)


EntryClass = Qwen3_5ForCausalLM

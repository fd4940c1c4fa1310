"""Qwen3 dense decoder (Qwen3ForCausalLM).

Computation order follows pymllm/models/qwen3.py:29-351: embedding -> N x
(RMSNorm with the residual add carried into it -> fused QKV projection -> per-head
RMSNorm of q and k -> NeoX RoPE -> attention over the KV pool -> o_proj ->
fused add + RMSNorm -> SwiGLU MLP) -> final norm -> last-token gather -> lm_head
(tied to the embedding when the config says so).  Checkpoint names are the HF
ones; q/k/v and gate/up are stacked into fused parameters by ``load_weights``.

Tensor parallelism: heads and MLP columns are split over the TP ranks (KV heads
are replicated when there are fewer than ranks); o_proj / down_proj are
row-parallel.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Iterable, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..engine.forward_batch import ForwardBatch
from ..layers import MLP, MergedLinear, RMSNorm, RadixAttention, RowParallelLinear, VocabParallelEmbedding
from ..parallel import state as pstate
from ..parallel.symm import get_tp_comm


class LogitsProcessorOutput:
    """Result of a forward pass.  ``next_token_logits`` are the full-vocabulary logits of the rows that
    produce a token; under tensor parallelism a pass may hand over only this rank's vocabulary slice
    (``local_logits`` + ``gather``), and the full logits are then assembled the first time they are asked for —
    greedy decoding never asks (``next_token_ids`` come from per-rank maxima and one tiny all-gather)."""

    def __init__(self, next_token_logits: Optional[torch.Tensor] = None, hidden_states: Optional[torch.Tensor] = None,
                 pp_placeholder: bool = False, local_logits: Optional[torch.Tensor] = None, gather=None) -> None:
        self._full = next_token_logits
        self.hidden_states = hidden_states
        # pipeline parallelism: on every stage but the last the logits are a [rows, 1] stand-in and the sampled
        # ids arrive from the last stage
        self.pp_placeholder = pp_placeholder
        self.local_logits, self._gather = local_logits, gather

    @property
    def next_token_logits(self) -> Optional[torch.Tensor]:
        if self._full is None and self.local_logits is not None:
            self._full = self._gather(self.local_logits)
        return self._full

    @next_token_logits.setter
    def next_token_logits(self, value: Optional[torch.Tensor]) -> None:
        self._full, self.local_logits = value, None


def _quant_method(quant_config, prefix: str):
    return quant_config.get_quant_method(None, prefix) if quant_config is not None else None


class Qwen3Attention(nn.Module):
    def __init__(self, config, layer_id: int, quant_config=None, prefix: str = "", params_dtype=None,
                 mrope_sections=None, mrope_interleaved: bool = False) -> None:
        super().__init__()
        tp = pstate.get_tensor_model_parallel_world_size()
        self.hidden_size = config.hidden_size
        self.total_heads = config.num_attention_heads
        self.total_kv_heads = config.num_key_value_heads
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        if self.total_heads % tp:
            raise ValueError(f"num_attention_heads={self.total_heads} not divisible by tp={tp}")
        self.num_heads = self.total_heads // tp
        kv_replicated = self.total_kv_heads < tp
        self.num_kv_heads = 1 if kv_replicated else self.total_kv_heads // tp
        self.kv_replicated = kv_replicated
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        eps = getattr(config, "rms_norm_eps", 1e-6)
        kv_width = self.kv_size if kv_replicated else self.total_kv_heads * self.head_dim
        self.qkv_proj = MergedLinear(
            self.hidden_size, [self.total_heads * self.head_dim, kv_width, kv_width],
            bias=getattr(config, "attention_bias", False), quant_method=_quant_method(quant_config, f"{prefix}.qkv_proj"),
            params_dtype=params_dtype, prefix=f"{prefix}.qkv_proj", shard_names=["q", "k", "v"],
            replicated_shards=[False, kv_replicated, kv_replicated],
        )
        self.o_proj = RowParallelLinear(self.total_heads * self.head_dim, self.hidden_size, bias=False,
                                        quant_method=_quant_method(quant_config, f"{prefix}.o_proj"),
                                        params_dtype=params_dtype, prefix=f"{prefix}.o_proj")
        # per-head RMSNorm of q and k: Qwen3 has it, the Llama / Qwen2 families (served by subclasses) do not
        self.use_qk_norm = bool(getattr(config, "use_qk_norm", True))
        if self.use_qk_norm:
            self.q_norm = RMSNorm(self.head_dim, eps, params_dtype)
            self.k_norm = RMSNorm(self.head_dim, eps, params_dtype)
        rope_theta = _rope_theta(config)
        self.attn = RadixAttention(self.num_heads, self.head_dim, self.head_dim ** -0.5, self.num_kv_heads, layer_id,
                                   rope_theta=rope_theta, rms_eps=eps, mrope_sections=mrope_sections,
                                   mrope_interleaved=mrope_interleaved, rope_scaling=_rope_scaling(config, layer_id),
                                   sliding_window=_sliding_window(config, layer_id),
                                   logit_cap=float(getattr(config, "attn_logit_softcapping", 0.0) or 0.0))

    def kv_shard_for_rank(self, loaded: torch.Tensor) -> torch.Tensor:
        """With fewer KV heads than ranks, rank r keeps head ``r * Hkv // tp``."""
        tp = pstate.get_tensor_model_parallel_world_size()
        r = pstate.get_tensor_model_parallel_rank()
        head = r * self.total_kv_heads // tp
        rows = loaded.shape[0] // self.total_kv_heads
        return loaded.narrow(0, head * rows, rows)

    def forward(self, x: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        qkv = self.qkv_proj(x)
        qw, kw = (self.q_norm.weight, self.k_norm.weight) if self.use_qk_norm else (None, None)
        a = self.attn(qkv, qw, kw, forward_batch)
        # under tensor parallelism the partial sums go to the next norm, which reduces them
        return self.o_proj.forward_partial(a) if self.o_proj.tp_size > 1 else self.o_proj(a)


def _rope_theta(config) -> float:
    theta = getattr(config, "rope_theta", None)
    if theta is None:
        rp = getattr(config, "rope_parameters", None) or getattr(config, "rope_scaling", None) or {}
        theta = rp.get("rope_theta", 1e6) if isinstance(rp, dict) else 1e6
    return float(theta)


def _rope_scaling(config, layer_id: int = 0) -> Optional[dict]:
    """The checkpoint's frequency rescaling (``rope_scaling`` / ``rope_parameters``) when it has one that
    changes the frequencies; M-RoPE sections are handled separately.  ``no_rope_layers`` (1 = rotate,
    0 = no positional rotation in that layer) turns the rotation off per layer."""
    use = getattr(config, "no_rope_layers", None)
    if use is not None and layer_id < len(use) and not use[layer_id]:
        return {"rope_type": "none"}
    rs = getattr(config, "rope_scaling", None) or getattr(config, "rope_parameters", None)
    if rs is None:
        return None
    rs = rs if isinstance(rs, dict) else vars(rs)
    kind = rs.get("rope_type", rs.get("type", "default"))
    if kind in (None, "default", "mrope"):
        return None
    if kind not in ("linear", "llama3", "yarn", "dynamic", "longrope"):
        raise NotImplementedError(f"rope scaling type {kind!r}")
    rs = dict(rs)
    # yarn / longrope also look at how far the context was stretched
    rs.setdefault("max_position_embeddings", getattr(config, "max_position_embeddings", None))
    if getattr(config, "original_max_position_embeddings", None):
        rs.setdefault("original_max_position_embeddings", config.original_max_position_embeddings)
    return rs


def _sliding_window(config, layer_id: int) -> Optional[int]:
    """The layer's attention window, if the checkpoint uses sliding-window attention: ``layer_types`` when
    given, else every layer (Mistral) or the layers from ``max_window_layers`` on (Qwen2 with
    ``use_sliding_window``)."""
    w = getattr(config, "sliding_window", None)
    if not w:
        return None
    types = getattr(config, "layer_types", None)
    if types:
        return int(w) if types[layer_id] == "sliding_attention" else None
    if hasattr(config, "use_sliding_window"):
        if not config.use_sliding_window:
            return None
        return int(w) if layer_id >= int(getattr(config, "max_window_layers", 0)) else None
    return int(w)


class Qwen3DecoderLayer(nn.Module):
    def __init__(self, config, layer_id: int, quant_config=None, prefix: str = "", params_dtype=None, **attn_kw):
        super().__init__()
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.self_attn = Qwen3Attention(config, layer_id, quant_config, f"{prefix}.self_attn", params_dtype, **attn_kw)
        self.mlp = self._make_mlp(config, layer_id, quant_config, f"{prefix}.mlp", params_dtype)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, params_dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, params_dtype)
        # the consumers of the two norms are plain tcgen05 GEMMs that can wait per gathered row tile
        from ..layers.quantize_base import UnquantizedLinearMethod

        self._gated_qkv = isinstance(self.self_attn.qkv_proj.quant_method, UnquantizedLinearMethod) and \
            self.self_attn.qkv_proj.bias is None
        self._gated_mlp = isinstance(self.mlp, MLP) and isinstance(self.mlp.gate_up_proj.quant_method, UnquantizedLinearMethod)
        self._plain_qkv = isinstance(self.self_attn.qkv_proj.quant_method, UnquantizedLinearMethod)

    def _make_mlp(self, config, layer_id, quant_config, prefix, params_dtype):
        return MLP(config.hidden_size, config.intermediate_size, quant_config, prefix, params_dtype)

    def _small_batch_fusable(self, hidden) -> bool:
        """A handful of rows on one GPU with 16-bit weights: both norms of the layer run inside the GEMMs that
        consume them (``ops.add_rmsnorm_linear``)."""
        if not (isinstance(hidden, torch.Tensor) and hidden.is_cuda and hidden.dim() == 2 and hidden.shape[0] <= 8):
            return False
        attn = self.self_attn
        return (type(attn).forward is Qwen3Attention.forward and attn.o_proj.tp_size == 1 and type(self.mlp) is MLP
                and self._plain_qkv and self._gated_mlp and getattr(self.mlp.gate_up_proj, "_gate_up_interleaved", False)
                and type(self.input_layernorm) is RMSNorm and type(self.post_attention_layernorm) is RMSNorm)

    def _forward_small_batch(self, hidden, residual, forward_batch):
        attn = self.self_attn
        qkv, residual = ops.add_rmsnorm_linear(hidden, residual, self.input_layernorm.weight, self.input_layernorm.eps,
                                               attn.qkv_proj.weight, bias=attn.qkv_proj.bias)
        qw, kw = (attn.q_norm.weight, attn.k_norm.weight) if attn.use_qk_norm else (None, None)
        a = attn.o_proj(attn.attn(qkv, qw, kw, forward_batch))
        h, residual = ops.add_rmsnorm_linear(a, residual, self.post_attention_layernorm.weight,
                                             self.post_attention_layernorm.eps, self.mlp.gate_up_proj.weight, swiglu=True)
        return self.mlp.down_proj(h), residual

    def forward(self, hidden: torch.Tensor, residual: Optional[torch.Tensor], forward_batch: ForwardBatch
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._small_batch_fusable(hidden):
            return self._forward_small_batch(hidden, residual, forward_batch)
        # residual-carry: the add of the previous block's output happens inside the next norm
        if residual is None:
            residual = hidden
            hidden = self.input_layernorm(hidden)
        else:
            hidden, residual = self.input_layernorm(hidden, residual, partial=self.self_attn.o_proj.tp_size > 1,
                                                    gated=self._gated_qkv)
        tp = self.self_attn.o_proj.tp_size > 1
        hidden = self.self_attn(hidden, forward_batch)
        hidden, residual = self.post_attention_layernorm(hidden, residual, partial=tp, gated=self._gated_mlp)
        hidden = self.mlp(hidden)  # partial sums again when tp > 1
        return hidden, residual


class Qwen3Model(nn.Module):
    layer_cls = Qwen3DecoderLayer

    def __init__(self, config, quant_config=None, prefix: str = "model", params_dtype=None, **attn_kw) -> None:
        super().__init__()
        self.config = config
        # Tied weights double as the (vocabulary-sharded) lm_head, so they stay sharded; an untied
        # input table is replicated under tensor parallelism: the lookup then needs no collective
        # and the decode step can be captured in a CUDA graph without library collectives inside.
        tied = bool(getattr(config, "tie_word_embeddings", False))
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, params_dtype, shard=tied)
        # pipeline parallelism: a stage builds (and loads) only its own run of layers; the others are empty
        # placeholders so that layer indices in parameter names stay global
        self.pp_layers = pstate.pp_layer_range(config.num_hidden_layers)
        self.layers = nn.ModuleList(
            self.layer_cls(config, i, quant_config, f"{prefix}.layers.{i}", params_dtype, **attn_kw)
            if i in self.pp_layers else nn.Identity()
            for i in range(config.num_hidden_layers)
        )
        self.norm = RMSNorm(config.hidden_size, getattr(config, "rms_norm_eps", 1e-6), params_dtype)

    def _sparse_blocks_can_shard(self, rows: int) -> bool:
        if not hasattr(self, "_sparse"):
            from ..layers.moe import SparseMoeBlock

            self._sparse = [m for m in self.modules() if isinstance(m, SparseMoeBlock)]
        return all(b.can_exchange(rows) for b in self._sparse)

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, forward_batch: ForwardBatch,
                input_embeds: Optional[torch.Tensor] = None, deepstack_embeds=None) -> torch.Tensor:
        staged = pstate.get_pipeline_parallel_world_size() > 1
        if not staged or pstate.pp_is_first_stage():
            hidden = self.embed_tokens(input_ids) if input_embeds is None else input_embeds
            residual = None
        else:
            # the block output of the previous stage (partial sums under TP) and its residual stream
            w = self.norm.weight
            hidden = pstate.pp_recv_prev(torch.empty((input_ids.shape[0], w.shape[0]), dtype=w.dtype, device=w.device))
            residual = pstate.pp_recv_prev(torch.empty_like(hidden))
        comm = get_tp_comm()
        if comm is not None:
            # deepstack injection adds to the block output, which the fused prefill step never materialises; a
            # sparse block can follow the row-sharded residual only through the expert-parallel exchange
            comm.prefill_fusion = deepstack_embeds is None and self._sparse_blocks_can_shard(input_ids.shape[0])
        for i in self.pp_layers:
            hidden, residual = self.layers[i](hidden, residual, forward_batch)
            if deepstack_embeds is not None and i < len(deepstack_embeds):
                # the MLP output is a partial sum under TP: inject on one rank only so it is counted once
                if pstate.get_tensor_model_parallel_rank() == 0:
                    hidden = hidden + deepstack_embeds[i]
        if staged and not pstate.pp_is_last_stage():
            pstate.pp_send_next(hidden)
            pstate.pp_send_next(residual)
            return None
        if residual is None:
            return self.norm(hidden)
        tp = pstate.get_tensor_model_parallel_world_size() > 1
        hidden, _ = self.norm(hidden, residual, partial=tp)
        return hidden


class Qwen3ForCausalLM(nn.Module):
    model_cls = Qwen3Model
    # (fused parameter, checkpoint name, shard id)
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", "q"),
        (".qkv_proj", ".k_proj", "k"),
        (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0),
        (".gate_up_proj", ".up_proj", 1),
    ]

    def __init__(self, config, quant_config=None, params_dtype: Optional[torch.dtype] = None, **model_kw) -> None:
        super().__init__()
        self.config = config
        self.quant_config = quant_config
        self.model = self.model_cls(config, quant_config, "model", params_dtype, **model_kw)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        if not self.tie:
            self.lm_head = VocabParallelEmbedding(config.vocab_size, config.hidden_size, params_dtype)
        self.tp_size = pstate.get_tensor_model_parallel_world_size()

    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.model.embed_tokens.weight if self.tie else self.lm_head.weight

    def compute_logits(self, hidden: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        if forward_batch.forward_mode.is_extend() and forward_batch.extend_seq_lens is not None:
            last = torch.cumsum(forward_batch.extend_seq_lens, 0) - 1
            hidden = hidden.index_select(0, last)
        logits = ops.linear(hidden, self.lm_head_weight)
        if self.tp_size > 1:
            if logits.is_cuda and torch.cuda.is_current_stream_capturing():
                return logits  # this rank's vocabulary slice; gathered by the caller after the replay
            logits = pstate.tensor_model_parallel_all_gather(logits, dim=-1)
        return logits[:, : self.config.vocab_size]

    def local_greedy(self, local_logits: torch.Tensor):
        """This rank's best candidate per row: (logit value fp32 [rows], global token id int64 [rows]); columns
        that only pad the vocabulary to a multiple of the rank count are left out."""
        per_rank = local_logits.shape[-1]
        start = pstate.get_tensor_model_parallel_rank() * per_rank if self.tp_size > 1 else 0
        valid = min(per_rank, self.config.vocab_size - start)
        if valid <= 0:      # this rank holds padding only
            rows = local_logits.shape[0]
            return (torch.full((rows,), float("-inf"), device=local_logits.device),
                    torch.zeros(rows, dtype=torch.int64, device=local_logits.device))
        vals, idx = local_logits[:, :valid].float().max(dim=-1)
        return vals, idx.to(torch.int64) + start

    def pick_greedy(self, vals: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """Global argmax from every rank's :meth:`local_greedy` candidates: one all-gather of two numbers per
        row; ties go to the lower token id, as a full-vocabulary argmax would decide."""
        if self.tp_size == 1:
            return ids
        pair = torch.stack([vals, ids.to(torch.float32)], dim=-1)                    # ids < 2^24: exact in fp32
        allp = pstate.tensor_model_parallel_all_gather(pair.unsqueeze(0), dim=0)     # [tp, rows, 2]
        best = allp[..., 0].argmax(dim=0)                                            # first rank holding the max
        return allp[..., 1].gather(0, best.unsqueeze(0)).squeeze(0).to(torch.int64)

    def gather_logits(self, local_logits: torch.Tensor) -> torch.Tensor:
        """Full-vocabulary logits from per-rank slices (used after a graph replay)."""
        if self.tp_size == 1:
            return local_logits
        return pstate.tensor_model_parallel_all_gather(local_logits, dim=-1)[:, : self.config.vocab_size]

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, forward_batch: ForwardBatch,
                input_embeds: Optional[torch.Tensor] = None) -> LogitsProcessorOutput:
        t0 = time.perf_counter()
        hidden = self.model(input_ids, positions, forward_batch, input_embeds)
        if hidden is None:   # not the last pipeline stage: the sampled ids will come from there
            rows = forward_batch.batch_size
            return LogitsProcessorOutput(next_token_logits=torch.zeros((rows, 1), device=input_ids.device), pp_placeholder=True)
        out = LogitsProcessorOutput(next_token_logits=self.compute_logits(hidden, forward_batch))
        ms = (time.perf_counter() - t0) * 1e3
        if forward_batch.forward_mode.is_decode():
            forward_batch.llm_decode_ms = ms
        else:
            forward_batch.llm_prefill_ms = ms
        return out

    # ------------------------------------------------------------------ loading
    @staticmethod
    def _canonical_name(name: str) -> Optional[str]:
        for old, new in (("model.language_model.", "model."), ("language_model.model.", "model."),
                         ("language_model.", "model.")):
            if name.startswith(old):
                name = new + name[len(old):]
                break
        if "rotary_emb.inv_freq" in name:
            return None
        return name

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        params = dict(self.named_parameters())
        loaded = set()
        for raw_name, tensor in weights:
            name = self._canonical_name(raw_name)
            if name is None or name.startswith("visual.") or name.startswith("model.visual."):
                continue
            if name.startswith("lm_head.") and self.tie:
                continue
            target, shard = name, None
            for fused, part, sid in self.stacked_params_mapping:
                if part in name:
                    cand = name.replace(part, fused)
                    if cand in params:
                        target, shard = cand, sid
                        break
            if target not in params:     # not kept on this rank / stage, or not part of this architecture
                continue
            p = params[target]
            if shard in ("k", "v"):
                attn = self._attn_of(target)
                if attn is not None and attn.kv_replicated:
                    tensor = attn.kv_shard_for_rank(tensor)
            loader = getattr(p, "weight_loader", None)
            if loader is None:
                p.data.copy_(tensor.reshape(p.shape))
            elif shard is None:
                loader(p, tensor)
            else:
                loader(p, tensor, shard)
            loaded.add(target)
        return loaded

    def _attn_of(self, param_name: str) -> Optional[Qwen3Attention]:
        parts = param_name.split(".")
        try:
            i = parts.index("layers")
            return self.model.layers[int(parts[i + 1])].self_attn
        except (ValueError, IndexError):
            return None


EntryClass = Qwen3ForCausalLM

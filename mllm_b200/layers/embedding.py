"""Vocabulary-sharded embedding table (pymllm/layers/embedding.py:15-160): each rank holds
``vocab/tp`` rows, looks up the ids it owns, zeroes the others and the partial results are summed."""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..parallel import state as pstate


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, params_dtype: Optional[torch.dtype] = None,
                 shard: bool = True) -> None:
        super().__init__()
        self.tp_rank = pstate.get_tensor_model_parallel_rank() if shard else 0
        self.tp_size = pstate.get_tensor_model_parallel_world_size() if shard else 1
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        # pad so every rank holds the same number of rows
        self.padded = -(-num_embeddings // self.tp_size) * self.tp_size
        self.per_rank = self.padded // self.tp_size
        self.vocab_start = self.tp_rank * self.per_rank
        self.vocab_end = self.vocab_start + self.per_rank
        self.weight = nn.Parameter(
            torch.zeros(self.per_rank, embedding_dim, dtype=params_dtype or torch.get_default_dtype()),
            requires_grad=False)
        self.weight.weight_loader = self.weight_loader

    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
        lo = self.vocab_start
        hi = min(self.vocab_end, loaded.shape[0])
        if hi > lo:
            param.data[: hi - lo].copy_(loaded[lo:hi])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return ops.embedding(ids, self.weight)
        if torch.cuda.is_available() and ids.is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("a vocabulary-sharded embedding lookup needs a collective and cannot be graph-captured")
        mask = (ids < self.vocab_start) | (ids >= self.vocab_end)
        local = torch.where(mask, torch.zeros_like(ids), ids - self.vocab_start)
        out = ops.embedding(local, self.weight)
        out.masked_fill_(mask.unsqueeze(-1), 0)
        return pstate.tensor_model_parallel_all_reduce(out)

"""Linear layers: replicated, column-parallel, row-parallel and merged (fused QKV / gate_up).

Sharding rules and loader behaviour follow pymllm/layers/linear.py:42-467:
column-parallel shards the output dimension, row-parallel the input dimension
(all-reduce after the GEMM, bias added once), and the merged layer stacks
several logical projections along the output dimension with a loader that
accepts shard ids ``"q"/"k"/"v"`` or integers and understands packed and
per-channel-scale parameters.  All compute goes through ``quant_method.apply``.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch
from torch import nn

from ..parallel import state as pstate
from .quantize_base import LinearMethodBase, UnquantizedLinearMethod


def _divide(a: int, b: int) -> int:
    if a % b:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def _narrow_for_rank(t: torch.Tensor, dim: int, rank: int, world: int) -> torch.Tensor:
    n = _divide(t.shape[dim], world)
    return t.narrow(dim, rank * n, n)


class LinearBase(nn.Module):
    def __init__(self, quant_method: Optional[LinearMethodBase], params_dtype: Optional[torch.dtype]) -> None:
        super().__init__()
        self.quant_method = quant_method or UnquantizedLinearMethod()
        self.params_dtype = params_dtype or torch.get_default_dtype()

    def _make_bias(self, n: int, loader) -> None:
        b = nn.Parameter(torch.zeros(n, dtype=self.params_dtype), requires_grad=False)
        b.weight_loader = loader
        b.output_dim = 0
        self.register_parameter("bias", b)


class Linear(LinearBase):
    """Replicated ``y = x W^T + b``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, quant_method=None,
                 params_dtype=None, prefix: str = "") -> None:
        super().__init__(quant_method, params_dtype)
        self.in_features, self.out_features, self.prefix = in_features, out_features, prefix
        self.quant_method.create_weights(self, in_features, [out_features], in_features, out_features,
                                         self.params_dtype, weight_loader=self.weight_loader)
        if bias:
            self._make_bias(out_features, self.weight_loader)
        else:
            self.bias = None

    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
        if param.dim() == 1 and loaded.dim() == 2 and loaded.shape[1] == 1:
            loaded = loaded.reshape(-1)
        if param.shape != loaded.shape:
            raise ValueError(f"{self.prefix}: shape {tuple(loaded.shape)} does not fit {tuple(param.shape)}")
        param.data.copy_(loaded)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.quant_method.apply(self, x, self.bias, residual)


class ColumnParallelLinear(LinearBase):
    """Output dimension split over the tensor-parallel ranks."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, gather_output: bool = False,
                 quant_method=None, params_dtype=None, prefix: str = "") -> None:
        super().__init__(quant_method, params_dtype)
        self.tp_rank = pstate.get_tensor_model_parallel_rank()
        self.tp_size = pstate.get_tensor_model_parallel_world_size()
        self.in_features, self.out_features, self.prefix = in_features, out_features, prefix
        self.gather_output = gather_output
        self.out_per_rank = _divide(out_features, self.tp_size)
        self.quant_method.create_weights(self, in_features, [self.out_per_rank], in_features, out_features,
                                         self.params_dtype, weight_loader=self.weight_loader)
        if bias:
            self._make_bias(self.out_per_rank, self.weight_loader)
        else:
            self.bias = None

    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
        out_dim = getattr(param, "output_dim", None)
        if out_dim is not None and self.tp_size > 1 and loaded.dim() > out_dim:
            loaded = _narrow_for_rank(loaded, out_dim, self.tp_rank, self.tp_size)
        if param.dim() == 1 and loaded.dim() == 2 and loaded.shape[1] == 1:
            loaded = loaded.reshape(-1)
        param.data.copy_(loaded.reshape(param.shape))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.quant_method.apply(self, x, self.bias)
        if self.gather_output and self.tp_size > 1:
            y = pstate.tensor_model_parallel_all_gather(y, dim=-1)
        return y


class RowParallelLinear(LinearBase):
    """Input dimension split over the tensor-parallel ranks; partial sums are all-reduced."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, reduce_results: bool = True,
                 quant_method=None, params_dtype=None, prefix: str = "") -> None:
        super().__init__(quant_method, params_dtype)
        self.tp_rank = pstate.get_tensor_model_parallel_rank()
        self.tp_size = pstate.get_tensor_model_parallel_world_size()
        self.in_features, self.out_features, self.prefix = in_features, out_features, prefix
        self.reduce_results = reduce_results
        self.in_per_rank = _divide(in_features, self.tp_size)
        self.quant_method.create_weights(self, self.in_per_rank, [out_features], in_features, out_features,
                                         self.params_dtype, weight_loader=self.weight_loader)
        if bias:
            self._make_bias(out_features, lambda p, w, shard_id=None: p.data.copy_(w))
        else:
            self.bias = None

    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
        in_dim = getattr(param, "input_dim", None)
        if in_dim is not None and self.tp_size > 1 and loaded.dim() > in_dim:
            n = param.shape[in_dim]
            loaded = loaded.narrow(in_dim, self.tp_rank * n, n)
        if param.dim() == 1 and loaded.dim() == 2 and loaded.shape[1] == 1:
            loaded = loaded.reshape(-1)
        param.data.copy_(loaded.reshape(param.shape))

    def forward_partial(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's partial sums, left for the following norm to reduce.  When peer-mapped buffers
        exist and the batch fits, the GEMM writes straight into one of them."""
        from ..parallel.symm import get_tp_comm

        comm = get_tp_comm()
        rows = x.numel() // x.shape[-1]
        if (comm is not None and x.is_cuda and self.bias is None and comm.prefill_eligible(rows)
                and isinstance(self.quant_method, UnquantizedLinearMethod) and self.out_features == comm.hidden):
            from .. import ops

            # prefill: the GEMM's epilogue scatters the tiles to the ranks that own the rows
            return ops.tp_gemm_reduce_scatter(x, self.weight, comm)
        buf = comm.partial_buffer(rows) if (comm is not None and x.is_cuda and self.bias is None) else None
        if buf is not None and isinstance(self.quant_method, UnquantizedLinearMethod):
            from .. import ops

            return ops.linear(x, self.weight, out=buf)
        y = self.quant_method.apply(self, x, self.bias if self.tp_rank == 0 else None)
        if buf is not None:
            buf.copy_(y.reshape(buf.shape))
            return buf
        return y

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.tp_size == 1 or not self.reduce_results:
            return self.quant_method.apply(self, x, self.bias, residual)
        # bias and residual enter once (rank 0), after which the partial sums are reduced
        lead = self.tp_rank == 0
        y = self.quant_method.apply(self, x, self.bias if lead else None, residual if lead else None)
        return pstate.tensor_model_parallel_all_reduce(y)


class MergedLinear(LinearBase):
    """Several projections of the same input stacked along the output dimension.

    ``output_sizes`` are the *global* widths of the logical projections; each is split
    over the tensor-parallel ranks, so the local weight is
    ``[sum(size_i / tp), in]``.  ``shard_names`` optionally names the shards (``"q"``,
    ``"k"``, ``"v"``); integer ids always work.
    """

    def __init__(self, in_features: int, output_sizes: Sequence[int], bias: bool = False, quant_method=None,
                 params_dtype=None, prefix: str = "", shard_names: Optional[Sequence[str]] = None,
                 replicated_shards: Optional[Sequence[bool]] = None) -> None:
        super().__init__(quant_method, params_dtype)
        self.tp_rank = pstate.get_tensor_model_parallel_rank()
        self.tp_size = pstate.get_tensor_model_parallel_world_size()
        self.in_features, self.prefix = in_features, prefix
        self.output_sizes = list(output_sizes)
        self.shard_names = list(shard_names) if shard_names else None
        # a shard may be replicated instead of split (KV heads when tp > num_kv_heads)
        self.replicated = list(replicated_shards) if replicated_shards else [False] * len(self.output_sizes)
        self.local_sizes = [s if rep else _divide(s, self.tp_size) for s, rep in zip(self.output_sizes, self.replicated)]
        self.out_features = sum(self.local_sizes)
        self.quant_method.create_weights(self, in_features, self.local_sizes, in_features, sum(self.output_sizes),
                                         self.params_dtype, weight_loader=self.weight_loader)
        if bias:
            self._make_bias(self.out_features, self.weight_loader)
        else:
            self.bias = None

    def _shard_index(self, shard_id: Union[int, str]) -> int:
        if isinstance(shard_id, int):
            return shard_id
        if self.shard_names and shard_id in self.shard_names:
            return self.shard_names.index(shard_id)
        raise KeyError(f"{self.prefix}: unknown shard id {shard_id!r}")

    def weight_loader(self, param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
        if shard_id is None:  # already-fused checkpoint tensor
            if param.shape == loaded.shape:
                param.data.copy_(loaded)
                return
            raise ValueError(f"{self.prefix}: fused tensor {tuple(loaded.shape)} != {tuple(param.shape)}")
        idx = self._shard_index(shard_id)
        out_dim = getattr(param, "output_dim", 0)
        # parameters that do not depend on the output dimension (e.g. weight_shape) are shared
        if getattr(param, "ignore_shard", False):
            param.data.copy_(loaded.reshape(param.shape))
            return
        pack = getattr(param, "pack_factor", 1) if getattr(param, "packed_dim", None) == out_dim else 1
        offset = sum(self.local_sizes[:idx]) // pack
        size = self.local_sizes[idx] // pack
        if loaded.dim() <= out_dim:
            raise ValueError(f"{self.prefix}: cannot shard a {loaded.dim()}-D tensor along dim {out_dim}")
        if not self.replicated[idx] and self.tp_size > 1:
            loaded = loaded.narrow(out_dim, self.tp_rank * size, size)
        if loaded.shape[out_dim] != size:
            raise ValueError(
                f"{self.prefix}: shard {shard_id!r} has {loaded.shape[out_dim]} rows, expected {size}")
        dst = param.data.narrow(out_dim, offset, size)
        if dst.dim() == 1 and loaded.dim() == 2 and loaded.shape[1] == 1:
            loaded = loaded.reshape(-1)
        dst.copy_(loaded.reshape(dst.shape))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.quant_method.apply(self, x, self.bias)

    def forward_swiglu(self, x: torch.Tensor) -> torch.Tensor:
        return self.quant_method.apply_swiglu(self, x)

"""Process-group bookkeeping for tensor / expert / data / pipeline parallelism.

One process drives one GPU.  Rank layout (same arithmetic as
pymllm/orchestrator/parallel_state.py:67-110): tensor-parallel groups are
contiguous rank ranges ``[i*tp, (i+1)*tp)``, data-parallel groups are strided
``range(i, world, world // dp)`` and pipeline groups are contiguous.  Expert
parallelism reuses the tensor-parallel ranks.  With ``world_size == 1`` nothing
is initialised and every query answers rank 0 of 1.

The groups are ordinary ``torch.distributed`` groups (NCCL on GPUs, gloo on
CPU); they carry bootstrap traffic, the NCCL baseline collectives and pipeline
send/recv.  The fused compute+collective kernels use the symmetric peer buffers
of :mod:`mllm_b200.parallel.symm` instead.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class GroupCoordinator:
    """A rank's view of one process group (pymllm/orchestrator/group_coordinator.py:8-104)."""

    ranks: List[int]
    group: Optional[dist.ProcessGroup]
    rank_in_group: int

    @property
    def world_size(self) -> int:
        return len(self.ranks)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world_size > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.world_size == 1:
            return t
        dim = dim % t.dim()
        if dim == 0:
            out = torch.empty((t.shape[0] * self.world_size, *t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
            return out
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=dim)

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over ranks and keep this rank's slice of dim 0 (which must divide evenly)."""
        if self.world_size == 1:
            return t
        out = torch.empty((t.shape[0] // self.world_size, *t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
        return out

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size > 1:
            dist.broadcast(t, src=self.ranks[src], group=self.group)
        return t

    def broadcast_object(self, obj, src: int = 0):
        if self.world_size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=self.ranks[src], group=self.group)
        return box[0]

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(group=self.group)


_SOLO = GroupCoordinator(ranks=[0], group=None, rank_in_group=0)
_TP: GroupCoordinator = _SOLO
_DP: GroupCoordinator = _SOLO
_PP: GroupCoordinator = _SOLO
_EP: GroupCoordinator = _SOLO
_INITIALISED = False


def init_distributed(backend: Optional[str] = None, timeout_s: Optional[float] = None) -> None:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun's variables)."""
    if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    kw = {}
    if timeout_s is not None:
        import datetime

        kw["timeout"] = datetime.timedelta(seconds=timeout_s)
    dist.init_process_group(backend=backend, **kw)


def initialize_model_parallel(tp_size: int = 1, dp_size: int = 1, pp_size: int = 1, ep_size: int = 1,
                              backend: Optional[str] = None) -> None:
    global _TP, _DP, _PP, _EP, _INITIALISED
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if tp_size * dp_size * pp_size != world:
        raise ValueError(f"tp({tp_size}) * dp({dp_size}) * pp({pp_size}) != world size {world}")
    if ep_size not in (1, tp_size):
        raise ValueError("expert parallelism reuses the tensor-parallel ranks: ep_size must be 1 or tp_size")

    def make(groups: List[List[int]]) -> GroupCoordinator:
        mine = None
        for ranks in groups:
            g = dist.new_group(ranks, backend=backend) if world > 1 and len(ranks) > 1 else None
            if rank in ranks:
                mine = GroupCoordinator(ranks=ranks, group=g, rank_in_group=ranks.index(rank))
        assert mine is not None
        return mine

    # Rank layout inside one replica: tensor-parallel ranks are adjacent, pipeline stages are tp_size apart
    # (rank = stage * tp_size + tp_rank); data-parallel replicas are tp_size * pp_size apart.
    _TP = make([list(range(i * tp_size, (i + 1) * tp_size)) for i in range(world // tp_size)])
    block = tp_size * pp_size
    _PP = make([[rep * block + t + s * tp_size for s in range(pp_size)] for rep in range(world // block) for t in range(tp_size)])
    _DP = make([[r + rep * block for rep in range(dp_size)] for r in range(block)])
    _EP = _TP if ep_size == tp_size else _SOLO
    _INITIALISED = True


def destroy_model_parallel() -> None:
    global _TP, _DP, _PP, _EP, _INITIALISED
    _TP = _DP = _PP = _EP = _SOLO
    _INITIALISED = False


def model_parallel_is_initialized() -> bool:
    return _INITIALISED


def get_tp_group() -> GroupCoordinator:
    return _TP


def get_dp_group() -> GroupCoordinator:
    return _DP


def get_pp_group() -> GroupCoordinator:
    return _PP


def get_ep_group() -> GroupCoordinator:
    return _EP


def get_pipeline_parallel_rank() -> int:
    return _PP.rank_in_group


def get_pipeline_parallel_world_size() -> int:
    return _PP.world_size


def pp_is_first_stage() -> bool:
    return _PP.rank_in_group == 0


def pp_is_last_stage() -> bool:
    return _PP.rank_in_group == _PP.world_size - 1


def pp_send_next(t: torch.Tensor) -> None:
    """Point-to-point send of ``t`` to the same tensor-parallel rank of the next pipeline stage."""
    dist.send(t.contiguous(), dst=_PP.ranks[_PP.rank_in_group + 1], group=_PP.group)


def pp_recv_prev(t: torch.Tensor) -> torch.Tensor:
    dist.recv(t, src=_PP.ranks[_PP.rank_in_group - 1], group=_PP.group)
    return t


def pp_layer_range(num_layers: int) -> range:
    """The layers this pipeline stage owns: contiguous, the first ``num_layers % stages`` stages get one more."""
    n, r = _PP.world_size, _PP.rank_in_group
    base, extra = divmod(num_layers, n)
    lo = r * base + min(r, extra)
    return range(lo, lo + base + (1 if r < extra else 0))


def get_tensor_model_parallel_rank() -> int:
    return _TP.rank_in_group


def get_tensor_model_parallel_world_size() -> int:
    return _TP.world_size


def tensor_model_parallel_all_reduce(t: torch.Tensor) -> torch.Tensor:
    return _TP.all_reduce(t)


def tensor_model_parallel_all_gather(t: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return _TP.all_gather(t, dim)


def data_parallel_all_reduce(t: torch.Tensor) -> torch.Tensor:
    return _DP.all_reduce(t)

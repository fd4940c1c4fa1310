"""The fused tensor-parallel prefill protocol over a fake transport: N ranks in one process, each with
its own symmetric heap, peer addresses resolved by hand.  The buffers, offsets and target addresses
are the ones the real launch code computes (``TPComm.from_heap``, ``ops.rs_inbox_targets``); the three
device steps are restated here in PyTorch with the kernels' index rules:

* GEMM epilogue with reduce-scatter (rank s): row tile ``tr`` belongs to ``owner = tr // tiles_per_rank``;
  the tile goes to the owner's inbox slot ``s`` at local tile ``tr % tiles_per_rank`` and, once stored,
  ``tile_flags[local_tile * 8 + s] = epoch`` on the owner;
* reduce + residual + RMSNorm + all-gather (owner r): waits for all ``tp`` flags of a local tile, sums
  the slots in rank order in fp32, adds its residual shard, normalises, stores the rows at
  ``r * own + row`` of every rank's gathered buffer and then sets ``gather_flags[r * tiles_per_rank + tile]``
  on every rank;
* the consumer may read row tile ``tr`` of its gathered buffer once ``gather_flags[tr] >= epoch``.

Checked for 2, 4 and 8 ranks, for batches smaller than the buffers' capacity, and over two epochs."""

import pytest
import torch

from mllm_b200 import ops
from mllm_b200.parallel.symm import SymmetricHeap, TPComm

H = 64
BASE_SHIFT = 40


class FakeFabric:
    def __init__(self, tp, max_rows, prefill_rows, dtype=torch.bfloat16):
        self.tp, self.dtype = tp, dtype
        nbytes = TPComm.heap_bytes(H, dtype, tp, max_rows, prefill_rows)
        self.heaps = [SymmetricHeap.local(nbytes, world=tp) for _ in range(tp)]
        for h in self.heaps:
            h.base_ptrs = [(r + 1) << BASE_SHIFT for r in range(tp)]
        self.comms = [TPComm.from_heap(self.heaps[r], H, dtype, "cpu", r, tp, max_rows, prefill_rows) for r in range(tp)]

    def view(self, ptr, shape, dtype):
        """The memory a peer address points at."""
        rank, off = (ptr >> BASE_SHIFT) - 1, ptr & ((1 << BASE_SHIFT) - 1)
        n = torch.empty((), dtype=dtype).element_size()
        for d in shape:
            n *= d
        assert 0 <= rank < self.tp and off + n <= self.heaps[rank].buf.numel(), "peer access outside the heap"
        return self.heaps[rank].buf[off:off + n].view(dtype).view(*shape)


def gemm_epilogue_reduce_scatter(fab, s, partial, epoch):
    comm = fab.comms[s]
    p = comm.prefill
    M = partial.shape[0]
    own_cap = p.inbox.shape[1]
    tiles_per_rank = M // 128 // fab.tp
    targets = ops.rs_inbox_targets(comm)
    for tr in range(M // 128):
        owner, local_tile = divmod(tr, tiles_per_rank)
        dst = fab.view(targets[owner], (own_cap, H), fab.dtype)
        dst[local_tile * 128:(local_tile + 1) * 128] = partial[tr * 128:(tr + 1) * 128]
        flags = fab.view(p.tile_flag_ptrs[owner], (own_cap // 128 * 8,), torch.int32)
        flags[local_tile * 8 + s] = epoch


def reduce_norm_all_gather(fab, r, residual_shard, weight, M, epoch, eps=1e-6):
    comm = fab.comms[r]
    p = comm.prefill
    tp, own = fab.tp, M // fab.tp
    tiles_per_rank = own // 128
    for tile in range(tiles_per_rank):
        assert all(int(p.tile_flags[tile * 8 + src]) >= epoch for src in range(tp)), "a tile was never delivered"
        rows = slice(tile * 128, (tile + 1) * 128)
        acc = torch.zeros(128, H)
        for src in range(tp):
            acc += p.inbox[src, rows].float()
        res = (acc + residual_shard[rows].float()).to(fab.dtype)
        residual_shard[rows] = res
        x = res.float()
        normed = (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.float()).to(fab.dtype)
        for dst in range(tp):
            full = fab.view(p.hidden_ptrs[dst], (p.rows_cap, H), fab.dtype)
            full[r * own + tile * 128: r * own + (tile + 1) * 128] = normed
        for dst in range(tp):
            gf = fab.view(p.gather_flag_ptrs[dst], (p.rows_cap // 128,), torch.int32)
            gf[r * tiles_per_rank + tile] = epoch


@pytest.mark.parametrize("tp,prefill_rows,M", [(2, 1024, 1024), (4, 2048, 1024), (8, 2048, 2048), (8, 4096, 1024)])
def test_fused_prefill_step_over_fake_transport(tp, prefill_rows, M):
    torch.manual_seed(tp * 1000 + M)
    fab = FakeFabric(tp, max_rows=256, prefill_rows=prefill_rows)
    assert all(c.prefill_eligible(M) for c in fab.comms)
    assert not fab.comms[0].prefill_eligible(M + 128) and not fab.comms[0].prefill_eligible(256)
    own = M // tp
    weight = (torch.rand(H) + 0.5).to(torch.bfloat16)
    residual = torch.randn(M, H).to(torch.bfloat16)
    shards = [residual[r * own:(r + 1) * own].clone() for r in range(tp)]
    expect_res = residual.clone()
    for epoch in (1, 2):
        partials = [torch.randn(M, H).to(torch.bfloat16) for _ in range(tp)]
        for s in range(tp):
            gemm_epilogue_reduce_scatter(fab, s, partials[s], epoch)
        for r in reversed(range(tp)):           # owners finish in any order
            reduce_norm_all_gather(fab, r, shards[r], weight, M, epoch)
        acc = torch.zeros(M, H)
        for s in range(tp):
            acc += partials[s].float()
        expect_res = (acc + expect_res.float()).to(torch.bfloat16)
        x = expect_res.float()
        expect = (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * weight.float()).to(torch.bfloat16)
        for r in range(tp):
            p = fab.comms[r].prefill
            assert torch.equal(p.hidden_full[:M], expect), f"rank {r} gathered rows differ"
            assert torch.equal(shards[r], expect_res[r * own:(r + 1) * own])
            assert bool((p.gather_flags[: M // 128] == epoch).all())
            assert bool((p.gather_flags[M // 128:] == 0).all())          # tiles beyond the batch are untouched
            assert bool((p.hidden_full[M:] == 0).all())
    assert all(h.check_guards() == [] for h in fab.heaps)       # nothing was written outside a buffer


def test_decode_buffers_alternate_and_resolve_on_every_rank():
    fab = FakeFabric(4, max_rows=256, prefill_rows=0)
    for r, comm in enumerate(fab.comms):
        a, b, c = comm.partial_buffer(8), comm.partial_buffer(8), comm.partial_buffer(8)
        assert a.data_ptr() != b.data_ptr() and a.data_ptr() == c.data_ptr()
        which = [i for i, sl in enumerate(comm.slots) if sl is comm.slot_of(a)][0]
        a.fill_(float(r + 1))
        # every rank's address for this rank's buffer lands on the same bytes
        for other in fab.comms:
            seen = fab.view(other.slots[which].data_ptrs[r], (256, H), torch.bfloat16)
            assert float(seen[0, 0]) == r + 1
        assert comm.partial_buffer(257) is None

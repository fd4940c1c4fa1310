"""CUDA-graph capture and replay of the decode step.

Batch-size schedule, capture order and padding policy follow
pymllm/executor/cuda_graph_runner.py:95-548: sizes
``[1, 2, 4, 8, 12, 16..256 step 8, 272..496 step 16, 512.. step 32]`` up to
``max_running_requests``; capture from the largest size down on a side stream, all graphs
sharing one memory pool; replay pads the batch up to the next captured size with rows that
point at the request table's spare row (``ReqToTokenPool.pad_row``, owned by no request) and KV slot 0
(the padding sink) and slices the outputs.

The whole step — embedding, every layer, lm_head and the greedy argmax — sits inside the
graph.  The attention kernels take sequence lengths and the request->slot table from
device memory, so replay needs no host-side planning: it is five small copies and one
``graph.replay()``.
"""

from __future__ import annotations

import bisect
import gc
import logging
from typing import Dict, List, Optional

import torch

from .. import ops
from ..engine.forward_batch import ForwardBatch, ForwardMode
from ..models.qwen3 import LogitsProcessorOutput

logger = logging.getLogger(__name__)


def capture_batch_sizes(max_bs: int) -> List[int]:
    sizes = [1, 2, 4, 8, 12] + list(range(16, 257, 8)) + list(range(272, 497, 16)) + list(range(512, max(513, max_bs + 1), 32))
    out = sorted({s for s in sizes if s <= max_bs})
    if not out or out[-1] < max_bs:
        out.append(max_bs)
    return out


class CudaGraphRunner:
    def __init__(self, model_runner, batch_sizes: Optional[List[int]] = None) -> None:
        self.mr = model_runner
        self.device = model_runner.device
        self.max_bs = model_runner.max_running_requests
        self.batch_sizes = batch_sizes or capture_batch_sizes(self.max_bs)
        n = self.batch_sizes[-1]
        dev = self.device
        # static inputs; padded rows use the request table's spare row / write KV slot 0
        self.pad_row = int(getattr(model_runner.req_to_token_pool, "pad_row", 0))
        self.input_ids = torch.zeros(n, dtype=torch.int64, device=dev)
        self.req_pool_indices = torch.full((n,), self.pad_row, dtype=torch.int32, device=dev)
        self.seq_lens = torch.ones(n, dtype=torch.int32, device=dev)
        self.out_cache_loc = torch.zeros(n, dtype=torch.int64, device=dev)
        self.positions = torch.zeros(n, dtype=torch.int64, device=dev)
        self.mrope_positions = torch.zeros((3, n), dtype=torch.int64, device=dev)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.logits: Dict[int, torch.Tensor] = {}
        self.next_ids: Dict[int, torch.Tensor] = {}
        self.kernels_per_graph: Dict[int, int] = {}
        self.pool = None
        self.replays = 0
        self.replayed_kernels = 0
        self.uses_mrope = bool(getattr(model_runner.model, "uses_mrope", False))
        self.tp_sharded_logits = getattr(model_runner.model, "tp_size", 1) > 1

    def _batch(self, bs: int) -> ForwardBatch:
        return ForwardBatch(
            forward_mode=ForwardMode.DECODE, batch_size=bs, input_ids=self.input_ids[:bs],
            req_pool_indices=self.req_pool_indices[:bs], seq_lens=self.seq_lens[:bs],
            out_cache_loc=self.out_cache_loc[:bs], positions=self.positions[:bs],
            max_seq_len=self.mr.context_len, req_to_token_pool=self.mr.req_to_token_pool,
            token_to_kv_pool=self.mr.token_to_kv_pool,
            mrope_positions=self.mrope_positions[:, :bs] if self.uses_mrope else None,
        )

    def _run(self, bs: int):
        fb = self._batch(bs)
        out = self.mr.model(fb.input_ids, fb.positions, fb)
        if self.tp_sharded_logits:
            # vocabulary slice: this rank's best candidate per row is found inside the graph; the ranks'
            # candidates are compared after the replay (full logits are gathered only if someone needs them)
            return out.next_token_logits, self.mr.model.local_greedy(out.next_token_logits)
        return out.next_token_logits, ops.argmax(out.next_token_logits)

    @torch.no_grad()
    def capture(self) -> None:
        gc.collect()
        gc.freeze()
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        try:
            with torch.cuda.stream(stream):
                for bs in reversed(self.batch_sizes):
                    for _ in range(2):  # warm-up: allocations and lazy initialisation happen here
                        self._run(bs)
                    torch.cuda.current_stream().synchronize()
                    before = ops.launch_count()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=self.pool, stream=stream):
                        logits, ids = self._run(bs)
                    self.kernels_per_graph[bs] = ops.launch_count() - before
                    if self.pool is None:
                        self.pool = g.pool()
                    self.graphs[bs], self.logits[bs], self.next_ids[bs] = g, logits, ids
        finally:
            gc.unfreeze()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        logger.info("captured %d decode graphs (batch sizes %s)", len(self.graphs), self.batch_sizes)

    def can_run(self, fb: ForwardBatch) -> bool:
        return fb.forward_mode.is_decode() and fb.batch_size <= self.batch_sizes[-1] and bool(self.graphs)

    def captured_size_for(self, raw: int) -> Optional[int]:
        """The captured batch size a batch of ``raw`` rows would replay, or None when none is large enough."""
        if not self.graphs or raw > self.batch_sizes[-1]:
            return None
        return self.batch_sizes[bisect.bisect_left(self.batch_sizes, raw)]

    @torch.no_grad()
    def replay_static(self, raw: int) -> LogitsProcessorOutput:
        """Replay for a batch whose inputs were already written into this runner's static buffers (``input_ids``,
        ``req_pool_indices``, ``seq_lens``, ``out_cache_loc``, ``positions``) by a kernel of the caller; rows past
        ``raw`` must hold the padding values (they do after construction and after any padded :meth:`replay`)."""
        bs = self.batch_sizes[bisect.bisect_left(self.batch_sizes, raw)]
        self.graphs[bs].replay()
        self.replays += 1
        self.replayed_kernels += self.kernels_per_graph.get(bs, 0)
        return self._outputs(bs, raw)

    def _outputs(self, bs: int, raw: int) -> LogitsProcessorOutput:
        if self.tp_sharded_logits:
            out = LogitsProcessorOutput(local_logits=self.logits[bs][:raw], gather=self.mr.model.gather_logits)
            vals, ids = self.next_ids[bs]
            out.next_token_ids = self.mr.model.pick_greedy(vals[:raw], ids[:raw])
            return out
        out = LogitsProcessorOutput(next_token_logits=self.logits[bs][:raw])
        out.next_token_ids = self.next_ids[bs][:raw]
        return out

    @torch.no_grad()
    def replay(self, fb: ForwardBatch) -> LogitsProcessorOutput:
        raw = fb.batch_size
        bs = self.batch_sizes[bisect.bisect_left(self.batch_sizes, raw)]
        if bs != raw:  # reset the padded tail
            self.req_pool_indices[raw:bs].fill_(self.pad_row)
            self.seq_lens[raw:bs].fill_(1)
            self.out_cache_loc[raw:bs].zero_()
            self.positions[raw:bs].zero_()
        self.input_ids[:raw].copy_(fb.input_ids, non_blocking=True)
        self.req_pool_indices[:raw].copy_(fb.req_pool_indices, non_blocking=True)
        self.seq_lens[:raw].copy_(fb.seq_lens, non_blocking=True)
        self.out_cache_loc[:raw].copy_(fb.out_cache_loc, non_blocking=True)
        self.positions[:raw].copy_(fb.positions, non_blocking=True)
        if self.uses_mrope and fb.mrope_positions is not None:
            self.mrope_positions[:, :raw].copy_(fb.mrope_positions, non_blocking=True)
        self.graphs[bs].replay()
        self.replays += 1
        self.replayed_kernels += self.kernels_per_graph.get(bs, 0)
        return self._outputs(bs, raw)

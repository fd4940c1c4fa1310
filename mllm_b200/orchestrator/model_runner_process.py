"""GPU-side request bookkeeping that sits between the scheduler and the ModelRunner.

Role of pymllm/orchestrator/model_runner_process.py:41-1166, with the same ownership rules:

* a request's row of ``req_to_token`` lists the KV slots of its tokens; the first ``prefix_len``
  of them belong to the radix tree (the request only *locks* them), the rest belong to the
  request until they are handed to the tree;
* prefill: match the prompt against the tree (page aligned), lock the matched node, take a request
  slot, allocate KV slots for the new tokens — evicting unlocked tree leaves and retrying when the
  pool is short — and write prefix + new slots into the request's row;
* after a prompt has been prefilled, and again when a request finishes, its (page-aligned) tokens
  are inserted into the tree: slots the tree already had are duplicates and are freed, the others
  change owner; the unaligned tail is freed when the request ends.

Additions over the reference: prompts can be prefilled in chunks (``extend`` takes any token range
of a request) and decode rows can ride along in an extend batch (a decode row is an extend of one
token), which is what the scheduler's chunked / mixed batches use.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..engine.sampling_params import SamplingParams
from ..executor.model_runner import ModelRunner, SamplingBatchInfo
from ..mem_cache import ChunkCache, MambaRadixCache, RadixCache, RadixKey

logger = logging.getLogger(__name__)


@dataclass
class Req:
    rid: str
    input_ids: List[int]
    sampling: SamplingParams
    stream: bool = False
    input_text: str = ""
    mm_inputs: Optional[Dict[str, Any]] = None
    extra_key: Optional[str] = None
    stop_token_ids: set = field(default_factory=set)
    stop_strs: List[str] = field(default_factory=list)   # generation ends when the text contains one of these
    created_time: float = 0.0
    # generation state
    output_ids: List[int] = field(default_factory=list)
    finished_reason: Optional[str] = None
    # cache state
    req_pool_idx: int = -1
    prefix_len: int = 0            # tokens whose KV belongs to the radix tree
    cached_tokens: int = 0         # prefix hit at admission (reported to the client)
    num_computed: int = 0          # tokens whose KV is in the pool (prefix + prefilled chunks + decoded)
    last_node: Any = None
    # page_size > 1: slots of the request's last page that are not used yet (pages are never shared)
    spare_slots: Any = None
    # timing (seconds, host clock)
    first_token_time: float = 0.0
    finish_time: float = 0.0
    last_stream_len: int = 0
    mrope_delta: int = 0
    # log-probabilities of the generated tokens (when the request asked for them)
    return_logprob: bool = False
    top_logprobs_num: int = 0
    output_logprobs: List[float] = field(default_factory=list)
    output_top_logprobs: List[List[Tuple[int, float]]] = field(default_factory=list)

    @property
    def seq_len(self) -> int:
        return len(self.input_ids) + len(self.output_ids)

    @property
    def finished(self) -> bool:
        return self.finished_reason is not None

    def all_ids(self) -> List[int]:
        return self.input_ids + self.output_ids

    def last_id(self) -> int:
        return self.output_ids[-1] if self.output_ids else self.input_ids[-1]


class KVAllocationError(RuntimeError):
    pass


def _make_radix_cache(alloc, page_size: int):
    """The C++ radix tree when the host extension is available (``MLLM_B200_PY_RADIX=1`` forces the
    Python tree, which has the same interface and eviction order)."""
    import os

    if os.environ.get("MLLM_B200_PY_RADIX") != "1":
        try:
            from ..mem_cache.native import NativeRadixCache

            return NativeRadixCache(alloc, page_size)
        except Exception as exc:  # extension not built on this machine
            logger.warning("native radix tree unavailable (%s); using the Python tree", exc)
    return RadixCache(alloc, page_size)


class ModelRunnerProcess:
    def __init__(self, runner: ModelRunner, disable_radix_cache: bool = False) -> None:
        self.runner = runner
        self.device = runner.device
        self.page_size = runner.server_config.radix_cache_page_size
        alloc = runner.token_to_kv_pool_allocator
        self.state_pool = getattr(runner, "gdn_pool", None)  # hybrid models: recurrent state per request row
        if disable_radix_cache:
            self.prefix_cache = ChunkCache(alloc, self.page_size)
        elif self.state_pool is not None:
            # a cached prefix of a hybrid model is reusable only where the recurrent state at its end was
            # kept: the state-aware tree when snapshot rows exist, no reuse otherwise
            self.prefix_cache = (MambaRadixCache(alloc, self.page_size, self.state_pool)
                                 if self.state_pool.track_slots > 0 else ChunkCache(alloc, self.page_size))
        else:
            self.prefix_cache = _make_radix_cache(alloc, self.page_size)
        self.hybrid_cache = isinstance(self.prefix_cache, MambaRadixCache)
        self.stats = {"prefix_hit_tokens": 0, "prefill_tokens": 0, "evicted_tokens": 0}

    # ------------------------------------------------------------------ capacity
    def available_tokens(self) -> int:
        return self.runner.token_to_kv_pool_allocator.available_size() + self.prefix_cache.evictable_size()

    def free_req_slots(self) -> int:
        return self.runner.req_to_token_pool.available_size()

    def _alloc_kv_with_eviction(self, n: int, host: bool = False):
        alloc = self.runner.token_to_kv_pool_allocator
        for attempt in range(4):
            out = alloc.alloc_host(n) if host else alloc.alloc(n)
            if out is not None:
                return out
            want = max(n, alloc.size // 10)
            res = self.prefix_cache.evict(want)
            self.stats["evicted_tokens"] += res.full_evicted
            if res.full_evicted == 0 and attempt > 0:
                break
        raise KVAllocationError(
            f"KV pool exhausted: need {n} slots, free {alloc.available_size()}, "
            f"evictable {self.prefix_cache.evictable_size()}, protected {self.prefix_cache.protected_size()}")

    def _alloc_rows(self, needs: Sequence[Tuple[Req, int]]) -> torch.Tensor:
        """KV slots for the next ``n`` tokens of each request, concatenated in order.

        With one-slot pages this is a single allocation.  With larger pages every request owns whole pages —
        the allocator frees a page as soon as one of its slots is freed, so a page shared by two requests
        would be recycled while the other still reads it: a request first uses up what is left of its last
        page (``spare_slots``) and then gets pages of its own."""
        if self.page_size == 1:
            return self._alloc_kv_with_eviction(sum(n for _, n in needs))
        P = self.page_size
        pages = []
        for req, n in needs:
            have = 0 if req.spare_slots is None else len(req.spare_slots)
            pages.append(max(0, -(-(n - have) // P)))
        fresh = self._alloc_kv_with_eviction(sum(pages) * P, host=True) if sum(pages) else np.empty(0, dtype=np.int64)
        out, off = [], 0
        for (req, n), k in zip(needs, pages):           # nothing above changed a request: a failed allocation leaves no trace
            mine = fresh[off : off + k * P]
            off += k * P
            have = req.spare_slots if req.spare_slots is not None else mine[:0]
            run = np.concatenate([have, mine]) if len(have) else mine
            out.append(run[:n])
            req.spare_slots = run[n:]
        loc = torch.from_numpy(np.ascontiguousarray(np.concatenate(out)))
        return loc if self.device.type == "cpu" else loc.pin_memory().to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ admission
    def admit(self, req: Req) -> None:
        """Give the request a row and attach the longest cached prefix of its prompt."""
        slots = self.runner.req_to_token_pool.alloc(1)
        if slots is None:
            raise KVAllocationError("no free request slot")
        req.req_pool_idx = slots[0]
        # never reuse the whole prompt: the last prompt token must be computed to get logits
        key = RadixKey(req.input_ids[: max(0, len(req.input_ids) - 1)], req.extra_key)
        if req.mm_inputs and req.mm_inputs.get("pixel_values") is not None:
            # image prompts are prefilled whole: the 3-D positions after an image depend on its grid
            key = RadixKey([], req.extra_key)
        m = self.prefix_cache.match_prefix(key)
        req.prefix_len = req.cached_tokens = req.num_computed = m.prefix_len
        req.last_node = m.last_node
        self.prefix_cache.inc_lock_ref(req.last_node)
        if m.prefix_len:
            self.runner.req_to_token_pool.req_to_token[req.req_pool_idx, : m.prefix_len] = torch.from_numpy(
                m.indices.astype(np.int32)).to(self.device, non_blocking=True)
            self.stats["prefix_hit_tokens"] += m.prefix_len
            if self.hybrid_cache:  # resume the recurrent layers from the snapshot taken at the prefix's end
                self.state_pool.copy(m.state_slot, req.req_pool_idx)

    # ------------------------------------------------------------------ forward passes
    def extend(self, items: Sequence[Tuple[Req, int]], sampling: bool = True):
        """Run new tokens of several requests in one pass.

        ``items``: (request, number of new tokens) — the tokens are the next ones after
        ``req.num_computed`` in ``prompt + generated``.  Returns (sampled ids or None, rows that
        produced a token): a row produces a token when its range ends at the current end of the
        request's sequence."""
        r = self.runner
        rtt = r.req_to_token_pool.req_to_token
        ids: List[int] = []
        ext_lens, pre_lens, pool_idx = [], [], []
        total = sum(n for _, n in items)
        loc = self._alloc_rows(items)
        off = 0
        for req, n in items:
            seq = req.all_ids()
            start = req.num_computed
            ids.extend(seq[start : start + n])
            rtt[req.req_pool_idx, start : start + n] = loc[off : off + n].to(torch.int32)
            off += n
            ext_lens.append(n)
            pre_lens.append(start)
            pool_idx.append(req.req_pool_idx)
        dev = self.device
        t_ids = torch.tensor(ids, dtype=torch.int64).to(dev, non_blocking=True)
        t_ext = torch.tensor(ext_lens, dtype=torch.int32).to(dev, non_blocking=True)
        t_pre = torch.tensor(pre_lens, dtype=torch.int32).to(dev, non_blocking=True)
        t_pool = torch.tensor(pool_idx, dtype=torch.int32).to(dev, non_blocking=True)
        extra = self._mm_kwargs(items)
        uses_mrope = bool(getattr(r.model, "uses_mrope", False))
        if uses_mrope:  # position offsets already known for continued requests
            extra["mrope_position_deltas"] = torch.tensor([q.mrope_delta for q, _ in items], dtype=torch.int64).to(dev)
        fb = r.prepare_forward_batch_extend(t_ids, t_pool, t_ext + t_pre, t_ext, t_pre, loc,
                                            extend_seq_lens_cpu=ext_lens, extend_prefix_lens_cpu=pre_lens, **extra)
        out = r.forward(fb)
        if uses_mrope and fb.mrope_position_deltas is not None:
            for (q, _), d in zip(items, fb.mrope_position_deltas.tolist()):
                q.mrope_delta = int(d)
        self.stats["prefill_tokens"] += total
        produced = []
        for i, (req, n) in enumerate(items):
            req.num_computed += n
            if req.num_computed == req.seq_len:
                produced.append(i)
        next_ids = None
        if sampling and produced:
            rows = torch.tensor(produced, device=dev)
            logits = out.next_token_logits.index_select(0, rows)
            out.next_token_logits = logits
            next_ids = r.sample(out, self._sampling_info([items[i][0] for i in produced]))
            self._record_logprobs([items[i][0] for i in produced], logits, next_ids)
        for i in produced:  # the prompt (and what was generated so far) becomes reusable
            req = items[i][0]
            if not req.output_ids:
                self._insert(req, req.input_ids)
        return next_ids, produced, fb

    def decode(self, reqs: Sequence[Req]):
        """One new token for every running request (graph path of the runner)."""
        r = self.runner
        dev = self.device
        bs = len(reqs)
        loc = self._alloc_rows([(q, 1) for q in reqs])
        pool = torch.tensor([q.req_pool_idx for q in reqs], dtype=torch.int32).to(dev, non_blocking=True)
        pos = torch.tensor([q.num_computed for q in reqs], dtype=torch.int64).to(dev, non_blocking=True)
        last = torch.tensor([q.last_id() for q in reqs], dtype=torch.int64).to(dev, non_blocking=True)
        r.req_to_token_pool.req_to_token[pool.long(), pos] = loc.to(torch.int32)
        seq_lens = (pos + 1).to(torch.int32)
        max_len = max(q.num_computed for q in reqs) + 1
        extra = {}
        if any(q.mrope_delta for q in reqs) or getattr(r.model, "uses_mrope", False):
            p1 = pos + torch.tensor([q.mrope_delta for q in reqs], dtype=torch.int64).to(dev, non_blocking=True)
            extra["mrope_positions"] = p1.unsqueeze(0).expand(3, -1).contiguous()
        fb = r.prepare_forward_batch_decode(last, pool, seq_lens, loc, max_seq_len=max_len, **extra)
        out = r.forward(fb)
        for q in reqs:
            q.num_computed += 1
        info = self._sampling_info(reqs)
        pre = getattr(out, "next_token_ids", None)
        if pre is not None and info.all_greedy and not info.has_penalties:
            nxt = pre
        else:
            nxt = r.sample(out, info)
        if any(q.return_logprob for q in reqs):      # touching the logits may trigger a cross-rank gather
            self._record_logprobs(reqs, out.next_token_logits, nxt)
        return nxt, fb

    @staticmethod
    def _record_logprobs(reqs: Sequence[Req], logits: torch.Tensor, next_ids: torch.Tensor) -> None:
        """For the requests that asked: log-probability of the sampled token (and the ``top_logprobs_num``
        most likely tokens) under the model's distribution — softmax of the logits the sampler saw,
        before temperature / top-k / top-p.  Row i of ``logits`` / ``next_ids`` belongs to ``reqs[i]``."""
        want = [i for i, q in enumerate(reqs) if q.return_logprob]
        if not want:
            return
        rows = torch.tensor(want, device=logits.device)
        lp = torch.log_softmax(logits.index_select(0, rows).float(), dim=-1)
        chosen = lp.gather(1, next_ids.index_select(0, rows).long().view(-1, 1)).view(-1).tolist()
        k = max(reqs[i].top_logprobs_num for i in want)
        top_v = top_i = None
        if k > 0:
            tv, ti = lp.topk(min(k, lp.shape[-1]), dim=-1)
            top_v, top_i = tv.tolist(), ti.tolist()
        for j, i in enumerate(want):
            q = reqs[i]
            q.output_logprobs.append(float(chosen[j]))
            n = q.top_logprobs_num
            q.output_top_logprobs.append([(int(top_i[j][c]), float(top_v[j][c])) for c in range(n)] if n > 0 else [])

    # ------------------------------------------------------------------ finish / cache
    def _insert(self, req: Req, tokens: List[int]) -> None:
        """Hand the KV of ``tokens`` (a prefix of the request's sequence, all computed) to the tree."""
        n = len(tokens) - len(tokens) % self.page_size
        n = min(n, req.num_computed)
        n -= n % self.page_size
        if n <= req.prefix_len or isinstance(self.prefix_cache, ChunkCache):
            return
        extra = {}
        if self.hybrid_cache:
            # the request's state row describes exactly `num_computed` tokens: only a prefix of that
            # length can be cached, and only if a snapshot row can be had for it
            snap = self.prefix_cache.alloc_state_slot() if n == req.num_computed else None
            if snap is None:
                return
            self.state_pool.copy(req.req_pool_idx, snap)
            extra["mamba_value"] = snap
        slots = self.runner.req_to_token_pool.req_to_token[req.req_pool_idx, :n].to("cpu", torch.int64).numpy()
        res = self.prefix_cache.insert(RadixKey(tokens[:n], req.extra_key), slots, **extra)
        # [prefix_len, res.prefix_len): the tree already had these tokens under other slots -> ours are duplicates
        if res.prefix_len > req.prefix_len:
            self.runner.token_to_kv_pool_allocator.free(slots[req.prefix_len : res.prefix_len])
            m = self.prefix_cache.match_prefix(RadixKey(tokens[:n], req.extra_key))
            self.runner.req_to_token_pool.req_to_token[req.req_pool_idx, : m.prefix_len] = torch.from_numpy(
                m.indices.astype(np.int32)).to(self.device, non_blocking=True)
            new_node = m.last_node
        else:
            new_node = res.last_node
        # move the lock from the old node to the node that now covers the inserted tokens
        self.prefix_cache.inc_lock_ref(new_node)
        self.prefix_cache.dec_lock_ref(req.last_node)
        req.last_node = new_node
        req.prefix_len = n

    def release(self, req: Req, cache: bool = True) -> None:
        """Request finished or aborted: give its KV to the tree (or free it) and free its row."""
        if req.req_pool_idx < 0:
            return
        if cache and req.num_computed > req.prefix_len:
            self._insert(req, req.all_ids()[: req.num_computed])
        tail = self.runner.req_to_token_pool.req_to_token[req.req_pool_idx, req.prefix_len : req.num_computed]
        if req.spare_slots is not None and len(req.spare_slots):
            # the unused rest of the last page goes back in the same call as the tail: the allocator returns a
            # page once per call in which one of its slots appears
            spare = torch.from_numpy(np.ascontiguousarray(req.spare_slots)).to(tail.dtype)
            tail = torch.cat([tail.to("cpu"), spare])
        req.spare_slots = None
        if tail.numel():
            self.runner.token_to_kv_pool_allocator.free(tail)
        self.prefix_cache.dec_lock_ref(req.last_node)
        self.runner.req_to_token_pool.free(req.req_pool_idx)
        req.req_pool_idx = -1
        req.last_node = None

    def flush_cache(self) -> bool:
        if self.prefix_cache.protected_size() > 0:
            return False
        self.prefix_cache.evict(self.prefix_cache.evictable_size())
        self.prefix_cache.reset()
        return True

    # ------------------------------------------------------------------ helpers
    def _sampling_info(self, reqs: Sequence[Req]) -> SamplingBatchInfo:
        dev = self.device
        all_greedy = all(q.sampling.is_greedy for q in reqs)
        any_pen = any(q.sampling.has_penalties for q in reqs)
        if all_greedy and not any_pen:
            return SamplingBatchInfo.greedy(len(reqs), dev)
        info = SamplingBatchInfo(
            temperatures=torch.tensor([0.0 if q.sampling.is_greedy else q.sampling.temperature for q in reqs], device=dev),
            top_ks=torch.tensor([q.sampling.top_k for q in reqs], dtype=torch.int32, device=dev),
            top_ps=torch.tensor([q.sampling.top_p for q in reqs], device=dev),
            min_ps=torch.tensor([q.sampling.min_p for q in reqs], device=dev),
            all_greedy=all_greedy,
        )
        if any_pen:
            V = self.runner.vocab_size
            counts = torch.zeros((len(reqs), V), dtype=torch.int32, device=dev)
            prompt = torch.zeros((len(reqs), V), dtype=torch.bool, device=dev)
            for i, q in enumerate(reqs):
                if q.output_ids:
                    counts[i] = torch.bincount(torch.tensor(q.output_ids, device=dev), minlength=V)[:V].int()
                prompt[i, torch.tensor(q.input_ids, device=dev).clamp_(0, V - 1)] = True
            info.output_counts, info.prompt_mask = counts, prompt
            info.frequency_penalties = torch.tensor([q.sampling.frequency_penalty for q in reqs], device=dev)
            info.presence_penalties = torch.tensor([q.sampling.presence_penalty for q in reqs], device=dev)
            info.repetition_penalties = torch.tensor([q.sampling.repetition_penalty for q in reqs], device=dev)
        seeds = [q.sampling.seed for q in reqs if q.sampling.seed is not None]
        if seeds:
            g = torch.Generator(device=dev)
            g.manual_seed(int(seeds[0]) + sum(len(q.output_ids) for q in reqs))
            info.generator = g
        return info

    def _mm_kwargs(self, items) -> Dict[str, Any]:
        """Pixel inputs of requests whose image tokens fall inside this pass."""
        pixel, grids, scales, scaled = [], [], [], False
        for req, _ in items:
            mm = req.mm_inputs
            if mm and mm.get("pixel_values") is not None and not mm.get("_consumed"):
                pixel.append(torch.as_tensor(mm["pixel_values"]))
                grids.append(torch.as_tensor(mm["image_grid_thw"]).reshape(-1, 3))
                if mm.get("mrope_t_scale") is not None:
                    scales.append(torch.as_tensor(mm["mrope_t_scale"], dtype=torch.float64).reshape(-1))
                    scaled = True
                else:
                    scales.append(torch.ones(grids[-1].shape[0], dtype=torch.float64))
                mm["_consumed"] = True
        if not pixel:
            return {}
        out = {"pixel_values": torch.cat(pixel).to(self.device), "image_grid_thw": torch.cat(grids).to(self.device)}
        if scaled:
            out["mrope_t_scale"] = torch.cat(scales)          # read on the host when positions are built
        return out

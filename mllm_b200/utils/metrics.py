"""Prometheus-style counters, gauges and histograms for the server (the reference declares
``enable_metrics`` but implements nothing behind it: pymllm/configs/server_config.py:85)."""

from __future__ import annotations

import threading
from collections import defaultdict
from typing import Any, Dict, List

_TTFT_BUCKETS = [0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0]
_TPOT_BUCKETS = [0.002, 0.004, 0.006, 0.008, 0.012, 0.02, 0.04, 0.08, 0.2]


class _Histogram:
    def __init__(self, buckets: List[float]) -> None:
        self.buckets = buckets
        self.counts = [0] * (len(buckets) + 1)
        self.total = 0.0
        self.n = 0

    def observe(self, v: float) -> None:
        self.n += 1
        self.total += v
        for i, b in enumerate(self.buckets):
            if v <= b:
                self.counts[i] += 1
                return
        self.counts[-1] += 1

    def render(self, name: str) -> List[str]:
        out, acc = [], 0
        for b, c in zip(self.buckets, self.counts):
            acc += c
            out.append(f'{name}_bucket{{le="{b}"}} {acc}')
        out.append(f'{name}_bucket{{le="+Inf"}} {self.n}')
        out += [f"{name}_sum {self.total}", f"{name}_count {self.n}"]
        return out


class Metrics:
    def __init__(self, enabled: bool = False) -> None:
        self.enabled = enabled
        self.lock = threading.Lock()
        self.http: Dict[str, int] = defaultdict(int)
        self.requests = 0
        self.prompt_tokens = 0
        self.completion_tokens = 0
        self.cached_tokens = 0
        self.ttft = _Histogram(_TTFT_BUCKETS)
        self.tpot = _Histogram(_TPOT_BUCKETS)
        self.gauges: Dict[str, float] = {}

    def observe_http(self, path: str, status: int, seconds: float) -> None:
        if self.enabled:
            with self.lock:
                self.http[f'{path}|{status}'] += 1

    def observe_request(self, meta: Dict[str, Any]) -> None:
        if not self.enabled:
            return
        with self.lock:
            self.requests += 1
            self.prompt_tokens += meta.get("prompt_tokens", 0)
            self.completion_tokens += meta.get("completion_tokens", 0)
            self.cached_tokens += meta.get("cached_tokens", 0)
            t = meta.get("timing")
            if t:
                self.ttft.observe(t["ttft_s"])
                if t["tpot_s"] > 0:
                    self.tpot.observe(t["tpot_s"])

    def sample_scheduler(self, sched) -> None:
        mrp = sched.mrp
        total = mrp.runner.max_total_num_tokens or 1
        free = mrp.runner.token_to_kv_pool_allocator.available_size()
        self.gauges = {
            "mllm_b200_queue_depth": len(sched.waiting), "mllm_b200_running_requests": len(sched.running),
            "mllm_b200_prefilling_requests": len(sched.prefilling), "mllm_b200_kv_usage_ratio": 1.0 - free / total,
            "mllm_b200_prefix_cache_tokens": mrp.prefix_cache.evictable_size() + mrp.prefix_cache.protected_size(),
            "mllm_b200_prefix_hit_tokens_total": mrp.stats["prefix_hit_tokens"],
            "mllm_b200_prefill_tokens_total": mrp.stats["prefill_tokens"],
        }

    def render(self) -> str:
        with self.lock:
            lines = [f"mllm_b200_requests_total {self.requests}", f"mllm_b200_prompt_tokens_total {self.prompt_tokens}",
                     f"mllm_b200_completion_tokens_total {self.completion_tokens}",
                     f"mllm_b200_cached_tokens_total {self.cached_tokens}"]
            for k, v in sorted(self.http.items()):
                path, status = k.split("|")
                lines.append(f'mllm_b200_http_requests_total{{path="{path}",status="{status}"}} {v}')
            lines += self.ttft.render("mllm_b200_ttft_seconds") + self.tpot.render("mllm_b200_tpot_seconds")
            lines += [f"{k} {v}" for k, v in sorted(self.gauges.items())]
        return "\n".join(lines) + "\n"

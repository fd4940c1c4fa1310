"""Serving benchmark.

Two workloads:

* ``--mode sequential`` — the reference's client (pymllm/bench_serve.py:52-395): for each prompt
  size one request at a time, ``--repeat`` times, reporting TTFT, TPOT (mean inter-token latency),
  end-to-end latency, prefill tokens/s and decode tokens/s; server-side ``debug_timing`` is used
  when the server provides it.
* ``--mode poisson`` — open-loop load: ``--num-requests`` requests arrive as a Poisson process of
  ``--request-rate`` requests/s; input lengths uniform in ``--input-len-range``, output lengths
  uniform in ``--output-len-range``; a ``--shared-prefix-ratio`` share of the requests starts with the
  same ``--shared-prefix-len`` random tokens (exercises radix prefix reuse).  Reports p50 / p90 / p99
  TTFT and TPOT, request and token throughput and the cached-token share.

Targets: an HTTP server (``--base-url``, OpenAI ``/v1/completions`` with SSE streaming) or an
in-process engine (``--engine``, any ``--server.*`` option applies), e.g.

    python -m mllm_b200.bench_serve --engine --server.model_path preset:qwen3-8b --mode poisson \
        --num-requests 512 --request-rate 16 --input-len-range 256 4096 --output-len-range 64 1024 \
        --shared-prefix-ratio 0.25 --shared-prefix-len 1024
"""

from __future__ import annotations

import argparse
import asyncio
import json
import random
import statistics
import sys
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class RequestResult:
    prompt_tokens: int
    output_tokens: int = 0
    cached_tokens: int = 0
    start: float = 0.0
    first_token: float = 0.0
    end: float = 0.0
    token_times: List[float] = field(default_factory=list)
    error: Optional[str] = None

    @property
    def ttft(self) -> float:
        return self.first_token - self.start

    @property
    def tpot(self) -> float:
        n = self.output_tokens
        return (self.end - self.first_token) / (n - 1) if n > 1 else 0.0

    @property
    def e2e(self) -> float:
        return self.end - self.start


def percentile(xs: List[float], p: float) -> float:
    if not xs:
        return 0.0
    xs = sorted(xs)
    k = (len(xs) - 1) * p / 100.0
    lo, hi = int(k), min(int(k) + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def make_workload(num: int, in_range, out_range, prefix_ratio: float, prefix_len: int, vocab: int, seed: int):
    """List of (prompt token ids, output length).  Deterministic for a seed."""
    rng = random.Random(seed)
    hi = max(2, min(vocab, 10000))
    shared = [rng.randrange(1, hi) for _ in range(prefix_len)]
    work = []
    for _ in range(num):
        n_in = rng.randint(*in_range)
        n_out = rng.randint(*out_range)
        if prefix_len and rng.random() < prefix_ratio and n_in > prefix_len:
            ids = shared + [rng.randrange(1, hi) for _ in range(n_in - prefix_len)]
        else:
            ids = [rng.randrange(1, hi) for _ in range(n_in)]
        work.append((ids, n_out))
    return work


def poisson_arrivals(num: int, rate: float, seed: int) -> List[float]:
    rng = random.Random(seed + 1)
    t, out = 0.0, []
    for _ in range(num):
        out.append(t)
        t += rng.expovariate(rate) if rate > 0 else 0.0
    return out


def summarize(results: List[RequestResult], wall: float) -> Dict[str, Any]:
    ok = [r for r in results if r.error is None and r.output_tokens > 0]
    ttft = [r.ttft for r in ok]
    tpot = [r.tpot for r in ok if r.output_tokens > 1]
    tot_in = sum(r.prompt_tokens for r in ok)
    tot_out = sum(r.output_tokens for r in ok)
    cached = sum(r.cached_tokens for r in ok)
    return {
        "completed": len(ok), "failed": len(results) - len(ok), "duration_s": wall,
        "first_error": next((r.error for r in results if r.error), None),
        "request_throughput": len(ok) / wall if wall else 0.0,
        "input_token_throughput": tot_in / wall if wall else 0.0,
        "output_token_throughput": tot_out / wall if wall else 0.0,
        "ttft_ms": {"mean": 1e3 * statistics.fmean(ttft) if ttft else 0.0, "p50": 1e3 * percentile(ttft, 50),
                    "p90": 1e3 * percentile(ttft, 90), "p99": 1e3 * percentile(ttft, 99)},
        "tpot_ms": {"mean": 1e3 * statistics.fmean(tpot) if tpot else 0.0, "p50": 1e3 * percentile(tpot, 50),
                    "p90": 1e3 * percentile(tpot, 90), "p99": 1e3 * percentile(tpot, 99)},
        "e2e_ms": {"p50": 1e3 * percentile([r.e2e for r in ok], 50), "p99": 1e3 * percentile([r.e2e for r in ok], 99)},
        "total_input_tokens": tot_in, "total_output_tokens": tot_out,
        "cached_token_ratio": cached / tot_in if tot_in else 0.0,
    }


# ------------------------------------------------------------------------------------------
# transports
# ------------------------------------------------------------------------------------------
async def _one_engine(engine, ids: List[int], n_out: int) -> RequestResult:
    from .engine.io_struct import GenerateReqInput

    r = RequestResult(prompt_tokens=len(ids), start=time.perf_counter())
    obj = GenerateReqInput(input_ids=ids, stream=True,
                           sampling_params={"max_new_tokens": n_out, "temperature": 0.0, "ignore_eos": True})
    try:
        async for o in engine.generate_async(obj):
            now = time.perf_counter()
            n = o["meta_info"]["completion_tokens"]
            if n > r.output_tokens:
                if r.output_tokens == 0:
                    r.first_token = now
                r.token_times.append(now)
                r.output_tokens = n
            r.cached_tokens = o["meta_info"].get("cached_tokens", 0)
    except Exception as exc:
        r.error = str(exc)
    r.end = time.perf_counter()
    return r


async def _one_http(session, base_url: str, ids: List[int], n_out: int, api_key: Optional[str]) -> RequestResult:
    r = RequestResult(prompt_tokens=len(ids), start=time.perf_counter())
    body = {"prompt": ids, "max_tokens": n_out, "temperature": 0.0, "stream": True, "ignore_eos": True,
            "stream_options": {"include_usage": True}}
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    try:
        async with session.post(f"{base_url}/v1/completions", json=body, headers=headers) as resp:
            if resp.status != 200:
                r.error = f"HTTP {resp.status}"
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                ev = json.loads(line[6:])
                now = time.perf_counter()
                if ev.get("error"):
                    r.error = str(ev["error"])[:200]
                elif ev.get("usage"):
                    r.output_tokens = max(r.output_tokens, ev["usage"]["completion_tokens"])
                    r.cached_tokens = ev["usage"].get("prompt_tokens_details", {}).get("cached_tokens", 0)
                elif ev.get("choices") and ev["choices"][0].get("text") is not None:
                    if r.first_token == 0.0:
                        r.first_token = now
                    r.token_times.append(now)
                    r.output_tokens += 1
    except Exception as exc:
        r.error = str(exc)
    r.end = time.perf_counter()
    return r


async def run_poisson(work, arrivals, engine=None, base_url=None, api_key=None) -> Dict[str, Any]:
    t0 = time.perf_counter()
    tasks = []
    session = None
    if engine is None:
        import aiohttp

        session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None))

    async def fire(delay, ids, n_out):
        await asyncio.sleep(max(0.0, delay - (time.perf_counter() - t0)))
        if engine is not None:
            return await _one_engine(engine, ids, n_out)
        return await _one_http(session, base_url, ids, n_out, api_key)

    for (ids, n_out), at in zip(work, arrivals):
        tasks.append(asyncio.ensure_future(fire(at, ids, n_out)))
    results = await asyncio.gather(*tasks)
    if session is not None:
        await session.close()
    return summarize(list(results), time.perf_counter() - t0)


async def run_sequential(prompt_sizes, out_len, repeat, vocab, seed, engine=None, base_url=None, api_key=None,
                         warmup: int = 0):
    rows = []
    session = None
    if engine is None:
        import aiohttp

        session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None))
    for w in range(max(0, warmup)):      # untimed requests: first-use costs (graphs, allocator, caches) stay out
        ids = make_workload(1, (prompt_sizes[0], prompt_sizes[0]), (8, 8), 0.0, 0, vocab, seed - 1 - w)[0][0]
        await (_one_engine(engine, ids, 8) if engine is not None else _one_http(session, base_url, ids, 8, api_key))
    for n_in in prompt_sizes:
        res = []
        for rep in range(repeat):
            ids = make_workload(1, (n_in, n_in), (out_len, out_len), 0.0, 0, vocab, seed + rep + n_in)[0][0]
            res.append(await (_one_engine(engine, ids, out_len) if engine is not None
                              else _one_http(session, base_url, ids, out_len, api_key)))
        ok = [r for r in res if r.error is None]
        if not ok:
            rows.append({"pp": n_in, "tg": out_len, "error": res[0].error})
            continue
        ttft = statistics.fmean(r.ttft for r in ok)
        tpot = statistics.fmean(r.tpot for r in ok)
        rows.append({"pp": n_in, "tg": out_len, "ttft_ms": ttft * 1e3, "tpot_ms": tpot * 1e3,
                     "e2e_ms": statistics.fmean(r.e2e for r in ok) * 1e3, "prefill_tok_s": n_in / ttft if ttft else 0.0,
                     "decode_tok_s": 1.0 / tpot if tpot else 0.0})
    if session is not None:
        await session.close()
    return rows


def print_report(rows) -> None:
    print(f"{'pp':>6} {'tg':>5} {'TTFT ms':>10} {'TPOT ms':>9} {'e2e ms':>10} {'prefill t/s':>12} {'decode t/s':>11}")
    for r in rows:
        if "error" in r:
            print(f"{r['pp']:>6} {r['tg']:>5}  error: {r['error']}")
        else:
            print(f"{r['pp']:>6} {r['tg']:>5} {r['ttft_ms']:>10.2f} {r['tpot_ms']:>9.3f} {r['e2e_ms']:>10.1f} "
                  f"{r['prefill_tok_s']:>12.1f} {r['decode_tok_s']:>11.1f}")


def main(argv=None) -> None:
    from .configs import make_args, read_args

    ap = argparse.ArgumentParser(prog="python -m mllm_b200.bench_serve")
    make_args(ap)
    ap.add_argument("--mode", choices=["sequential", "poisson"], default="sequential")
    ap.add_argument("--base-url", "--url", dest="base_url", default=None)
    # spelled as in the reference's bench_serve (llama-bench style pp / tg run against a live server)
    ap.add_argument("--prefill-sizes", dest="prompt_sizes", type=lambda v: [int(x) for x in str(v).split(",") if x],
                    help="comma-separated prompt sizes (same as --prompt-sizes)")
    ap.add_argument("--decode-tokens", dest="output_len", type=int, help="same as --output-len")
    ap.add_argument("--warmup", type=int, default=2, help="untimed requests before the sequential measurement")
    ap.add_argument("--temperature", type=float, default=0.0, help="accepted for compatibility; requests are greedy")
    ap.add_argument("--model", default=None, help="accepted for compatibility; the server serves one model")
    ap.add_argument("--client-timing", action="store_true",
                    help="accepted for compatibility: timings are always taken at the client from the token stream")
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--engine", action="store_true", help="drive an in-process engine instead of HTTP")
    ap.add_argument("--prompt-sizes", type=int, nargs="+", default=[128, 512, 2048])
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--num-requests", type=int, default=512)
    ap.add_argument("--request-rate", type=float, default=16.0)
    ap.add_argument("--input-len-range", type=int, nargs=2, default=[256, 4096])
    ap.add_argument("--output-len-range", type=int, nargs=2, default=[64, 1024])
    ap.add_argument("--shared-prefix-ratio", type=float, default=0.25)
    ap.add_argument("--shared-prefix-len", type=int, default=1024)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output-file", default=None)
    ap.add_argument("--vocab-size", type=int, default=10000,
                    help="HTTP mode: synthetic prompt ids are drawn below this (the served model's vocabulary must hold them)")
    ns = ap.parse_args(argv)
    cfg = read_args(argv, ap)
    engine = None
    vocab = ns.vocab_size
    if ns.engine:
        from .engine.launch import Engine

        engine = Engine(cfg, mode="inproc").launch()
        vocab = engine.scheduler.mrp.runner.vocab_size
    elif not ns.base_url:
        ns.base_url = f"http://{cfg.server.host}:{cfg.server.port}"
    try:
        if ns.mode == "sequential":
            rows = asyncio.run(run_sequential(ns.prompt_sizes, ns.output_len, ns.repeat, vocab, ns.seed, engine,
                                              ns.base_url, ns.api_key, warmup=ns.warmup))
            print_report(rows)
            result: Any = rows
        else:
            work = make_workload(ns.num_requests, tuple(ns.input_len_range), tuple(ns.output_len_range),
                                 ns.shared_prefix_ratio, ns.shared_prefix_len, vocab, ns.seed)
            arrivals = poisson_arrivals(ns.num_requests, ns.request_rate, ns.seed)
            result = asyncio.run(run_poisson(work, arrivals, engine, ns.base_url, ns.api_key))
            print(json.dumps(result, indent=1))
        if ns.output_file:
            with open(ns.output_file, "a") as f:
                f.write(json.dumps(result) + "\n")
    finally:
        if engine is not None:
            engine.shutdown()


if __name__ == "__main__":
    main()

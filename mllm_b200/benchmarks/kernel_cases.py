"""Small, self-contained launches of single kernels for profiling and micro-timing.

    python -m mllm_b200.benchmarks.kernel_cases attn_decode --batch 16 --seq 2050
    python -m mllm_b200.benchmarks.kernel_cases gemm --m 8 --n 4096 --k 12288
    python -m mllm_b200.benchmarks.kernel_cases attn_prefill --batch 2 --seq 2048

Each case allocates inputs larger than the 126 MB L2 where the kernel is memory bound, runs a
few warm-up launches, then times `--iters` launches with CUDA events and prints one JSON line
(algorithmic bytes / FLOPs and the achieved rates).  The cases are kept small (well under a few
GB) so that a profiler capture of one or two launches ends quickly.
"""

from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from ..ops import reference as ref


def _time(fn, iters: int, warm: int = 3) -> float:
    """Mean device time of one call: `iters` calls are captured into a CUDA graph and the graph is
    replayed between two events, so host launch cost does not enter the number."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(iters):
                fn()
    torch.cuda.current_stream().wait_stream(stream)
    graph.replay()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def _kv(batch, seq, hkv, dev):
    slots = batch * seq + 16
    kc = torch.randn(slots, hkv, 128, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(slots, hkv, 128, device=dev, dtype=torch.bfloat16)
    rtt = torch.zeros(batch, seq + 8, dtype=torch.int32, device=dev)
    rtt[:, :seq] = (torch.arange(batch * seq, device=dev, dtype=torch.int32) + 1).view(batch, seq)
    req = torch.arange(batch, dtype=torch.int32, device=dev)
    return kc, vc, rtt, req


def attn_decode(a) -> dict:
    dev = "cuda"
    kc, vc, rtt, req = _kv(a.batch, a.seq, a.hkv, dev)
    seq = torch.full((a.batch,), a.seq, dtype=torch.int32, device=dev)
    q = torch.randn(a.batch, a.hq, 128, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    ms = _time(lambda: ops.attention_decode(q, kc, vc, rtt, req, seq, 128 ** -0.5, out=out, max_seq_len=a.seq), a.iters)
    byts = 2 * a.batch * a.seq * a.hkv * 128 * 2
    return {"case": "attn_decode", "batch": a.batch, "seq": a.seq, "hq": a.hq, "hkv": a.hkv, "ms": ms,
            "gbs": byts / ms / 1e6}


def attn_prefill(a) -> dict:
    dev = "cuda"
    kc, vc, rtt, req = _kv(a.batch, a.seq, a.hkv, dev)
    seq = torch.full((a.batch,), a.seq, dtype=torch.int32, device=dev)
    pre = torch.zeros_like(seq)
    q = torch.randn(a.batch * a.seq, a.hq, 128, device=dev, dtype=torch.bfloat16)
    qs = (torch.arange(a.batch, device=dev, dtype=torch.int32) * a.seq)
    out = torch.empty_like(q)
    ms = _time(lambda: ops.attention_prefill(q, kc, vc, rtt, req, seq, pre, qs, 128 ** -0.5, out=out, max_q_len=a.seq), a.iters)
    flops = 4 * a.batch * a.hq * 128 * a.seq * a.seq / 2
    return {"case": "attn_prefill", "batch": a.batch, "seq": a.seq, "hq": a.hq, "hkv": a.hkv, "ms": ms,
            "tflops": flops / ms / 1e9}


def gemm(a) -> dict:
    dev = "cuda"
    x = torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16)
    # several weight copies so consecutive launches do not hit L2
    copies = max(1, min(8, int(3e8 // (a.n * a.k * 2)) + 1)) if a.m <= 256 else 1
    ws = [torch.randn(a.n, a.k, device=dev, dtype=torch.bfloat16) * a.k ** -0.5 for _ in range(copies)]
    if a.swiglu:
        ws = [ref.interleave_gate_up(w, ops.SWIGLU_BLOCK).contiguous() for w in ws]
    state = {"i": 0}

    def run():
        w = ws[state["i"] % copies]
        state["i"] += 1
        return ops.linear_swiglu(x, w) if a.swiglu else ops.linear(x, w)

    ms = _time(run, a.iters)
    byts = (a.n * a.k + a.m * a.k + a.m * a.n) * 2
    return {"case": "gemm", "m": a.m, "n": a.n, "k": a.k, "swiglu": a.swiglu, "ms": ms,
            "tflops": 2 * a.m * a.n * a.k / ms / 1e9, "gbs": byts / ms / 1e6}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["attn_decode", "attn_prefill", "gemm"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2050)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    out = {"attn_decode": attn_decode, "attn_prefill": attn_prefill, "gemm": gemm}[a.case](a)
    ops.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()

"""Small, self-contained launches of single kernels for profiling and micro-timing.

    python -m mllm_b200.benchmarks.kernel_cases attn_decode --batch 16 --seq 2050
    python -m mllm_b200.benchmarks.kernel_cases gemm --m 8 --n 4096 --k 12288
    python -m mllm_b200.benchmarks.kernel_cases attn_prefill --batch 2 --seq 2048
    python -m mllm_b200.benchmarks.kernel_cases gdn --batch 1 --seq 2048 --gdn-backend cuda_chunkwise

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
    # stored head-major like the KV pool, handed out as [slots, kv heads, 128] views
    kc = torch.randn(hkv, slots, 128, device=dev, dtype=torch.bfloat16).transpose(0, 1)
    vc = torch.randn(hkv, slots, 128, device=dev, dtype=torch.bfloat16).transpose(0, 1)
    rtt = torch.zeros(batch, seq + 8, dtype=torch.int32, device=dev)
    rtt[:, :seq] = (torch.arange(batch * seq, device=dev, dtype=torch.int32) + 1).view(batch, seq)
    req = torch.arange(batch, dtype=torch.int32, device=dev)
    return kc, vc, rtt, req


def attn_decode(a) -> dict:
    dev = "cuda"
    # several KV sets used in turn (like the layers of a model) so the working set exceeds L2
    sets = [_kv(a.batch, a.seq, a.hkv, dev) for _ in range(max(1, a.kv_sets))]
    seq = torch.full((a.batch,), a.seq, dtype=torch.int32, device=dev)
    q = torch.randn(a.batch, a.hq, 128, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)

    def run():
        for kc, vc, rtt, req in sets:
            ops.attention_decode(q, kc, vc, rtt, req, seq, 128 ** -0.5, out=out, max_seq_len=a.seq)

    ms = _time(run, a.iters) / len(sets)
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

    if a.param:
        ws = [torch.nn.Parameter(w, requires_grad=False) for w in ws]

    def run():
        w = ws[state["i"] % copies]
        state["i"] += 1
        if a.library:
            return torch.matmul(x, w.t())
        return ops.linear_swiglu(x, w) if a.swiglu else ops.linear(x, w)

    ms = _time(run, a.iters)
    byts = (a.n * a.k + a.m * a.k + a.m * a.n) * 2
    return {"case": "gemm", "m": a.m, "n": a.n, "k": a.k, "swiglu": a.swiglu, "library": a.library, "param": a.param, "ms": ms,
            "tflops": 2 * a.m * a.n * a.k / ms / 1e9, "gbs": byts / ms / 1e6}


def moe(a) -> dict:
    """Qwen3-30B-A3B-shaped expert block on one rank: hidden 2048, expert width 768, top-8 of 128 experts,
    ``--experts`` of them local (16 = one of eight expert-parallel ranks)."""
    dev = "cuda"
    H, I, E, k = 2048, 768, a.experts, 8
    x = torch.randn(a.m, H, device=dev, dtype=torch.bfloat16)
    w13 = torch.stack([ref.interleave_gate_up(torch.randn(2 * I, H, device=dev, dtype=torch.bfloat16) * H ** -0.5,
                                              ops.SWIGLU_BLOCK) for _ in range(E)]).contiguous()
    w2 = (torch.randn(E, H, I, device=dev, dtype=torch.bfloat16) * I ** -0.5).contiguous()
    logits = torch.randn(a.m, 128, device=dev, dtype=torch.bfloat16)
    tw = torch.empty(a.m, k, dtype=torch.float32, device=dev)
    ti = torch.empty(a.m, k, dtype=torch.int32, device=dev)
    ops.ext().moe_router_topk(logits, tw, ti, True)
    ms = _time(lambda: ops.moe_experts(x, w13, w2, tw, ti, 0, ops.SWIGLU_BLOCK, num_experts_global=128), a.iters)
    local_pairs = int((ti < E).sum())
    flops = 2 * local_pairs * 3 * I * H
    return {"case": "moe", "tokens": a.m, "local_experts": E, "local_pairs": local_pairs, "ms": ms,
            "tflops": flops / ms / 1e9, "weight_gbs": E * 3 * I * H * 2 / ms / 1e6}


def w4a16(a) -> dict:
    dev = "cuda"
    g = 128
    x = torch.randn(a.m, a.k, device=dev, dtype=torch.bfloat16)
    copies = max(1, min(8, int(3e8 // (a.n * a.k // 2)) + 1)) if a.m <= 256 else 1
    qws = [torch.randint(-(2 ** 31), 2 ** 31 - 1, (a.n, a.k // 8), device=dev, dtype=torch.int64).to(torch.int32)
           for _ in range(copies)]
    sc = (torch.rand(a.n, a.k // g, device=dev) * 0.02 + 0.005).to(torch.bfloat16)
    state = {"i": 0}

    def run():
        w = qws[state["i"] % copies]
        state["i"] += 1
        return ops.w4a16_gemm(x, w, sc, None, g)

    ms = _time(run, a.iters)
    return {"case": "w4a16", "m": a.m, "n": a.n, "k": a.k, "ms": ms, "tflops": 2 * a.m * a.n * a.k / ms / 1e9,
            "weight_gbs": a.n * a.k / 2 / ms / 1e6}


def gdn(a) -> dict:
    """Prefill of the gated delta rule: `--batch` requests of `--seq` new tokens, `--hq` heads of 128 x 128."""
    dev = "cuda"
    B, L, H, D = a.batch, a.seq, a.hq, 128
    T = B * L
    q, k, v = (torch.randn(T, H, D, device=dev).bfloat16() for _ in range(3))
    g = -torch.rand(T, H, device=dev) * 0.3
    beta = torch.rand(T, H, device=dev)
    slots = torch.arange(B, device=dev, dtype=torch.int32)
    lens = torch.full((B,), L, device=dev, dtype=torch.int32)
    has = torch.zeros(B, device=dev, dtype=torch.int32)
    st = torch.zeros(B, H, D, D, device=dev)
    ops.set_gdn_extend_backend(a.gdn_backend)
    ms = _time(lambda: ops.gated_delta_rule(q, k, v, g, beta, st, slots, lens, has), a.iters)
    ops.set_gdn_extend_backend("auto")
    # per token and head: S^T k, the rank-one update and S^T q touch the 128 x 128 state three times
    return {"case": "gdn", "backend": a.gdn_backend, "batch": B, "seq": L, "heads": H, "ms": ms,
            "us_per_64_tokens": ms * 1e3 / (L / 64), "state_tflops": 6 * T * H * D * D / ms / 1e9}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["attn_decode", "attn_prefill", "gemm", "moe", "w4a16", "gdn"])
    ap.add_argument("--gdn-backend", default="auto", choices=["auto", "cuda_chunkwise", "mllm_kernel"],
                    help="gdn: chunk-parallel kernel, token-sequential kernel, or the default choice between them")
    ap.add_argument("--experts", type=int, default=16, help="moe: local experts")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2050)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--library", action="store_true",
                    help="gemm: time the vendor library's GEMM (torch.matmul) on the same operands instead, for comparison")
    ap.add_argument("--param", action="store_true", help="gemm: hold the weights in an nn.Parameter (model-weight path)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--kv-sets", type=int, default=4, help="attn_decode: KV caches used in turn (working set > L2)")
    a = ap.parse_args()
    out = {"attn_decode": attn_decode, "attn_prefill": attn_prefill, "gemm": gemm, "moe": moe, "w4a16": w4a16, "gdn": gdn}[a.case](a)
    ops.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()

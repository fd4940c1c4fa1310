"""Device-timed pieces of one tensor-parallel prefill half-layer, fused vs collective-library path.

Run with one process per GPU, e.g.
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m mllm_b200.benchmarks.tp_prefill_cases``.
Prints (rank 0, max over ranks) the mean time of: the row-parallel GEMM alone, the GEMM with the
reduce-scatter epilogue, the reduce-scatter + add + RMSNorm + all-gather kernel (including the wait for
the gather), and all-reduce + add + RMSNorm through the process group."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--k-total", type=int, default=12288, help="input width of the row-parallel GEMM before sharding")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()

    from mllm_b200 import ops
    from mllm_b200.parallel import state as pstate
    from mllm_b200.parallel.symm import TPComm, set_tp_comm

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}")
    torch.cuda.set_device(dev)
    pstate.init_distributed(backend="nccl", timeout_s=120)
    pstate.initialize_model_parallel(tp_size=world)
    comm = TPComm.create(args.hidden, torch.bfloat16, dev, max_rows=256, prefill_rows=args.rows)
    assert comm is not None and comm.prefill_eligible(args.rows), "symmetric memory or shape not available"
    set_tp_comm(comm)
    M, H, K = args.rows, args.hidden, args.k_total // world
    g = torch.Generator(device=dev).manual_seed(rank)
    x = (torch.randn(M, K, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    w = (torch.randn(H, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    res_full = torch.zeros(M, H, device=dev, dtype=torch.bfloat16)
    res_shard = torch.zeros(M // world, H, device=dev, dtype=torch.bfloat16)
    names = ["gemm_plain", "gemm_rs", "rs_norm_ag", "allreduce_add_norm"]
    acc = {n: 0.0 for n in names}

    def timed(name, fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b.record()
        return name, a, b, r

    for it in range(args.iters + 3):
        dist.barrier()
        torch.cuda.synchronize()
        recs = []
        recs.append(timed("gemm_plain", lambda: ops.linear(x, w)))
        y = recs[-1][3]
        recs.append(timed("allreduce_add_norm", lambda: ops.tp_reduce_add_rmsnorm(y, res_full, nw, 1e-6)))
        recs.append(timed("gemm_rs", lambda: ops.tp_gemm_reduce_scatter(x, w, comm)))
        part = recs[-1][3]
        recs.append(timed("rs_norm_ag", lambda: ops.tp_rs_add_rmsnorm_ag(part, res_shard, nw, 1e-6, comm, gated=False)))
        torch.cuda.synchronize()
        if it >= 3:
            for name, a, b, _ in recs:
                acc[name] += a.elapsed_time(b)
    # decode-sized pieces: the fused peer-memory reduce + add + RMSNorm of 8 rows against the process group's
    # all-reduce followed by the local add + norm, 20 calls each inside one pair of events
    names += ["decode_reduce_fused", "decode_reduce_library"]
    rows_d = 8
    resid = torch.zeros(rows_d, H, device=dev, dtype=torch.bfloat16)
    yd = torch.randn(rows_d, H, device=dev, dtype=torch.bfloat16)
    for name in names[-2:]:
        for rep in range(2):                      # first repetition warms up
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(20):
                if name == "decode_reduce_fused":
                    part = comm.partial_buffer(rows_d)
                    part.copy_(yd)
                    ops.tp_reduce_add_rmsnorm(part, resid, nw, 1e-6)
                else:
                    tmp = yd.clone()
                    dist.all_reduce(tmp)
                    ops.fused_add_rmsnorm(tmp, resid, nw, 1e-6)
            b.record()
            torch.cuda.synchronize()
            acc[name] = a.elapsed_time(b) / 20 * args.iters    # per call; includes the 16 KB staging copy of both arms
    ops.check_status()
    t = torch.tensor([acc[n] / args.iters for n in names], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        out = {n: round(float(v), 4) for n, v in zip(names, t.tolist())}
        out.update(rows=M, hidden=H, k_per_rank=K, tp=world, unit="ms")
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

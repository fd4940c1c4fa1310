"""Step-by-step bring-up check of the tensor-parallel transport on N GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m mllm_b200.benchmarks.tp_selftest [--rows 2048] [--hidden 4096] [--deadline-s 240]

Each stage prints one line per rank when it completes (stage name, seconds since start), so a run that
stalls shows where; past the deadline every rank dumps its Python stacks and exits with status 3.  The
stages, in order: process group (gloo barrier, then an NCCL all-reduce), symmetric heap (one rendezvous,
canary bytes checked at the end), one fused decode reduce with a known answer, one fused prefill step
(GEMM with reduce-scatter epilogue -> reduce + add + RMSNorm + all-gather -> gated consumer GEMM) checked
against the collective-library path, and the kernels' status word.  Sizes are small: the whole check holds
well under a gigabyte per GPU and takes seconds once the processes are up."""

from __future__ import annotations

import argparse
import faulthandler
import json
import os
import sys
import threading
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048, help="prefill rows (rounded up to a multiple of 128 * ranks)")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--deadline-s", type=float, default=240.0)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    t0 = time.perf_counter()
    stage = {"name": "start"}
    done = threading.Event()

    def watchdog() -> None:
        if done.wait(args.deadline_s):
            return
        print(f"[tp_selftest rank {rank}] stuck in stage '{stage['name']}' after {args.deadline_s:.0f} s", file=sys.stderr, flush=True)
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        os._exit(3)

    threading.Thread(target=watchdog, daemon=True).start()

    def passed(name: str, **info) -> None:
        stage["name"] = name + " (done)"
        print(json.dumps({"rank": rank, "stage": name, "t_s": round(time.perf_counter() - t0, 2), **info}), flush=True)

    def enter(name: str) -> None:
        stage["name"] = name

    import torch
    import torch.distributed as dist

    from mllm_b200 import ops
    from mllm_b200.parallel import state as pstate
    from mllm_b200.parallel.symm import TPComm, set_tp_comm

    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    enter("process group")
    import datetime

    dist.init_process_group("cpu:gloo,cuda:nccl", timeout=datetime.timedelta(seconds=max(60.0, args.deadline_s)))
    host = torch.zeros(1)
    dist.all_reduce(host)
    passed("gloo barrier")
    enter("nccl all-reduce")
    t = torch.full((1024,), float(rank + 1), device=dev)
    dist.all_reduce(t)
    torch.cuda.synchronize()
    assert float(t[0]) == world * (world + 1) / 2
    passed("nccl all-reduce")
    pstate.initialize_model_parallel(tp_size=world)

    enter("symmetric heap")
    tp = world
    rows = (args.rows + 128 * tp - 1) // (128 * tp) * (128 * tp)
    while rows <= 256:          # the fused prefill path serves batches larger than the decode buffers
        rows += 128 * tp
    comm = TPComm.create(args.hidden, torch.bfloat16, dev, max_rows=256, prefill_rows=rows)
    if comm is None:
        passed("symmetric heap", available=False)
        done.set()
        dist.destroy_process_group()
        return
    set_tp_comm(comm)
    passed("symmetric heap", bytes=int(comm.heap.buf.numel()))

    enter("fused decode reduce")
    part = comm.partial_buffer(8)
    part.fill_(float(rank + 1))
    resid = torch.zeros(8, args.hidden, dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize()
    dist.all_reduce(host)
    ops.tp_reduce_add_rmsnorm(part, resid, None, 1e-6)
    torch.cuda.synchronize()
    ops.check_status(dev.index)
    assert bool((resid.float() == world * (world + 1) / 2).all()), "fused decode reduce gave a wrong sum"
    passed("fused decode reduce")

    enter("fused prefill step")
    H, K = args.hidden, 512
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = (torch.randn(rows, K, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    w = (torch.randn(H, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    g2 = torch.Generator(device=dev).manual_seed(7)
    w2 = (torch.randn(256, H, device=dev, generator=g2) * 0.02).to(torch.bfloat16)      # same on every rank
    # collective-library path
    y = ops.linear(x, w)
    dist.all_reduce(y)
    want_res = y.clone()
    want = ops.linear(ops.rmsnorm(want_res, nw, 1e-6), w2)
    # fused path
    own = rows // tp
    res_shard = torch.zeros(own, H, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    dist.all_reduce(host)
    token = ops.tp_gemm_reduce_scatter(x, w, comm)
    hidden_full, res_shard = ops.tp_rs_add_rmsnorm_ag(token, res_shard, nw, 1e-6, comm, gated=True)
    got = ops.linear(hidden_full, w2)          # consumer GEMM: waits per row tile for the gather
    torch.cuda.synchronize()
    ops.check_status(dev.index)
    err = (got.float() - want.float()).abs().max().item()
    scale = want.float().abs().max().item()
    res_err = (res_shard.float() - want_res[rank * own:(rank + 1) * own].float()).abs().max().item()
    assert err <= 0.05 * scale + 0.05 and res_err <= 0.1, (err, scale, res_err)
    passed("fused prefill step", rows=rows, max_abs_err=round(err, 4))

    enter("canaries")
    dist.all_reduce(host)
    torch.cuda.synchronize()
    assert comm.heap.check_guards() == [], "a kernel wrote outside a symmetric buffer"
    passed("canaries")
    done.set()
    dist.all_reduce(host)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

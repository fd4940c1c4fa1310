"""Step-by-step bring-up check of the tensor-parallel transport on N GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m mllm_b200.benchmarks.tp_selftest [--rows 8192] [--k-per-rank 512] [--hidden 4096] [--deadline-s 240]

Each stage prints one line per rank when it completes (stage name, seconds since start), so a run that
stalls shows where; past the deadline every rank dumps its Python stacks and exits with status 3.  The
stages, in order: process group (gloo barrier, then an NCCL all-reduce), symmetric heap (one rendezvous,
canary bytes checked at the end), one fused decode reduce with a known answer, one fused prefill step
(GEMM with reduce-scatter epilogue -> reduce + add + RMSNorm + all-gather -> gated consumer GEMM), several
times in a row, checked against an fp32 statement of the same sums, and the kernels' status word.  Sizes are small: the whole check holds
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
    ap.add_argument("--rows", type=int, default=8192, help="prefill rows (rounded up to a multiple of 128 * ranks)")
    ap.add_argument("--k-per-rank", type=int, default=512, help="reduction length of the row-parallel GEMM on one rank")
    ap.add_argument("--steps", type=int, default=3, help="fused prefill steps in a row")
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
    # random partials, residual and norm weight against fp32: the kernel sums the 16-bit partials in fp32 in
    # rank order, so the new residual is exact up to its own final rounding
    for rows_d in (1, 8, 64, 256):
        g = torch.Generator(device=dev).manual_seed(50 + rank + rows_d)
        part = comm.partial_buffer(rows_d)
        part.copy_((torch.randn(rows_d, args.hidden, device=dev, generator=g)).to(torch.bfloat16))
        g2 = torch.Generator(device=dev).manual_seed(9 + rows_d)
        resid = torch.randn(rows_d, args.hidden, device=dev, generator=g2).to(torch.bfloat16)
        nw = (1.0 + 0.1 * torch.randn(args.hidden, device=dev, generator=g2)).to(torch.bfloat16)
        total = part.float().clone()
        dist.all_reduce(total)
        want_res = (total + resid.float()).bfloat16().float()
        want = want_res * torch.rsqrt(want_res.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
        torch.cuda.synchronize()
        dist.all_reduce(host)
        out = ops.tp_reduce_add_rmsnorm(part, resid, nw, 1e-6)
        torch.cuda.synchronize()
        ops.check_status(dev.index)
        ulp = 2.0 ** -8 * want_res.abs() + 1e-6
        assert bool(((resid.float() - want_res).abs() <= ulp).all()), f"decode reduce: residual off ({rows_d} rows)"
        rel = ((out.float() - want).norm() / want.norm()).item()
        assert rel < 4e-3, (rows_d, rel)
    passed("fused decode reduce")

    enter("fused prefill step")
    # Several fused steps in a row (each has its own epoch), with enough 128-row tiles per CTA of the
    # reduce-scatter GEMM (rows x hidden / (128 x 256) tiles over ~148 CTAs) that the epilogue runs ahead of
    # the publisher thread.  Checked against an fp32 statement of the same mathematics: every rank's partial
    # product in fp32, summed in fp32, then add + RMSNorm in fp32.  The kernels round each rank's partial to
    # 16 bits before it crosses NVLink, so the bound on the residual stream is 2^-8 of the summed magnitudes.
    H, K = args.hidden, args.k_per_rank
    own = rows // tp
    worst = {"res": 0.0, "hidden": 0.0, "out": 0.0}
    for it in range(args.steps):
        g = torch.Generator(device=dev).manual_seed(1000 * it + 100 + rank)
        x = (torch.randn(rows, K, device=dev, generator=g) * 0.5).to(torch.bfloat16)
        w = (torch.randn(H, K, device=dev, generator=g) * K ** -0.5).to(torch.bfloat16)
        g2 = torch.Generator(device=dev).manual_seed(7 + it)              # same on every rank
        nw = (1.0 + 0.1 * torch.randn(H, device=dev, generator=g2)).to(torch.bfloat16)
        w2 = (torch.randn(2048, H, device=dev, generator=g2) * H ** -0.5).to(torch.bfloat16)   # enough tiles for the two-CTA tiling
        res0 = (torch.randn(rows, H, device=dev, generator=g2) * 0.5).to(torch.bfloat16)
        # fp32 statement
        part = x.float() @ w.float().t()
        mag = part.abs()
        dist.all_reduce(part)
        dist.all_reduce(mag)
        want_res = part + res0.float()
        want_hidden = want_res * torch.rsqrt(want_res.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
        want_out = want_hidden.bfloat16().float() @ w2.float().t()
        # fused path
        res_shard = res0[rank * own:(rank + 1) * own].clone()
        torch.cuda.synchronize()
        dist.all_reduce(host)
        token = ops.tp_gemm_reduce_scatter(x, w, comm)
        hidden_full, res_shard = ops.tp_rs_add_rmsnorm_ag(token, res_shard, nw, 1e-6, comm, gated=True)
        got = ops.linear(hidden_full, w2)          # consumer GEMM: waits per row tile for the gather
        torch.cuda.synchronize()
        ops.check_status(dev.index)
        sl = slice(rank * own, (rank + 1) * own)
        bound = 2.0 ** -8 * (mag[sl] + want_res[sl].abs()) + 1e-3
        excess = ((res_shard.float() - want_res[sl]).abs() - bound).max().item()
        assert excess <= 0.0, f"residual shard off by {excess} beyond the rounding bound (step {it})"
        rel_h = ((hidden_full.float() - want_hidden).norm(dim=-1) / want_hidden.norm(dim=-1).clamp_min(1e-6)).max().item()
        rel_o = ((got.float() - want_out).norm() / want_out.norm()).item()
        assert rel_h < 8e-3 and rel_o < 8e-3, (rel_h, rel_o, it)
        worst["res"] = max(worst["res"], ((res_shard.float() - want_res[sl]).abs() / bound).max().item())
        worst["hidden"], worst["out"] = max(worst["hidden"], rel_h), max(worst["out"], rel_o)
        del part, mag, want_res, want_hidden, want_out
    passed("fused prefill step", rows=rows, k_per_rank=K, steps=args.steps, epochs=int(comm.epoch),
           residual_err_over_bound=round(worst["res"], 3), hidden_rel_err=round(worst["hidden"], 5),
           out_rel_err=round(worst["out"], 5))

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

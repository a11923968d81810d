"""Device-timed micro-benchmarks of the communication kernels against NCCL, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m cosmos_b200.parallel.bench_comm [--mb 256] [--iters 10]

  * all-gather by pull (`allgather_pull`, FSDP parameter gather) vs `all_gather_into_tensor`
  * reduce-scatter by pull into an fp32 shard (`reduce_scatter_pull`, peer loads and multimem.ld_reduce) vs
    `reduce_scatter_tensor`
  * decode all-reduce + residual + RMS-norm in one kernel (`allreduce_norm`, both ways) vs NCCL all-reduce + the norm kernel

Every number is the maximum over ranks of a CUDA-event time (median of `--iters` runs after warm-up, a device barrier
before each timed launch so that the ranks start together). Bandwidths count the bytes that cross NVLink per rank:
(N - 1) / N of the buffer for gather and reduce-scatter. Rank 0 prints one JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def _time(fn, iters, pre=None):
    for _ in range(3):
        if pre:
            pre()
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if pre:
            pre()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256, help="size of the full (gathered / reduced) bf16 buffer in MiB")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from .. import ops
    from .symm import symm_group
    ops.load_extension()
    sg = symm_group(dist.group.WORLD, list(range(world)), dev)
    k = torch.ops.cosmos_b200

    def out(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    n = args.mb * (1 << 20) // 2
    n -= n % (world * 1024)
    ns = n // world
    link_bytes = (world - 1) / world * n * 2

    # ---- all-gather by pull
    sbuf = sg.alloc("bench_shard", ns * 2)
    shard = sbuf.view(0, (ns,), torch.bfloat16)
    shard.normal_()
    sptrs = torch.tensor(sbuf.peer_ptrs, dtype=torch.int64, device=dev)
    full = torch.empty(n, dtype=torch.bfloat16, device=dev)
    sg.barrier_host()
    ms = _time(lambda: k.allgather_pull(sptrs, world, full, ns * 2), args.iters)
    ms_n = _time(lambda: dist.all_gather_into_tensor(full, shard), args.iters)
    out(kernel="allgather_pull", ranks=world, mib=args.mb, ms=round(ms, 4), gbs_per_rank=round(link_bytes / ms / 1e6, 1),
        nccl_ms=round(ms_n, 4), nccl_gbs_per_rank=round(link_bytes / ms_n / 1e6, 1))

    # ---- reduce-scatter by pull
    gbuf = sg.alloc("bench_grad", n * 2)
    grad = gbuf.view(0, (n,), torch.bfloat16)
    grad.normal_()
    gptrs = torch.tensor(gbuf.peer_ptrs, dtype=torch.int64, device=dev)
    red = torch.empty(ns, dtype=torch.float32, device=dev)
    sq = torch.zeros(1, dtype=torch.float32, device=dev)
    sg.barrier_host()
    modes = [("peer loads", 0)]
    if sg.use_multicast(gbuf):
        modes.append(("multimem.ld_reduce", sg.use_multicast(gbuf)))
    nccl_out = torch.empty(ns, dtype=torch.bfloat16, device=dev)
    ms_n = _time(lambda: dist.reduce_scatter_tensor(nccl_out, grad), args.iters)
    for name, mc in modes:
        ms = _time(lambda: k.reduce_scatter_pull(gptrs, mc, world, rank * ns, red, False, 1.0 / world, sq), args.iters)
        out(kernel=f"reduce_scatter_pull ({name})", ranks=world, mib=args.mb, ms=round(ms, 4),
            gbs_per_rank=round(link_bytes / ms / 1e6, 1), nccl_ms=round(ms_n, 4),
            nccl_gbs_per_rank=round(link_bytes / ms_n / 1e6, 1))

    # ---- decode all-reduce + residual + RMS-norm
    m_rows, d = 32, 4096
    gamma = torch.ones(d, dtype=torch.bfloat16, device=dev)
    resid = torch.randn(m_rows, d, device=dev).bfloat16()
    bufs = []
    for i in range(2):
        b = sg.alloc(f"bench_arn_{i}", m_rows * d * 2)
        v = b.view(0, (m_rows, d), torch.bfloat16)
        v.normal_()
        bufs.append((v, torch.tensor(b.peer_ptrs, dtype=torch.int64, device=dev), sg.use_multicast(b)))
    sg.barrier_host()
    state = {"i": 0}

    def arn(use_mc):
        state["i"] ^= 1
        own, ptrs, mc = bufs[state["i"]]
        k.allreduce_norm(ptrs, mc if use_mc else 0, own, sg.pads_dev, rank, world, 16, sg.counters, m_rows, d, resid, gamma,
                         1e-6, True)

    x = torch.randn(m_rows, d, device=dev).bfloat16()

    def nccl_arn():
        y = x.clone()
        dist.all_reduce(y)
        ops.rmsnorm(y, gamma, 1e-6, residual=resid)

    # many calls per timed region: a single call is a few microseconds
    reps = 50
    ms_n = _time(lambda: [nccl_arn() for _ in range(reps)], args.iters) / reps
    for name, use_mc in [("peer loads", False)] + ([("multimem.ld_reduce", True)] if bufs[0][2] else []):
        ms = _time(lambda: [arn(use_mc) for _ in range(reps)], args.iters, pre=lambda: sg.barrier_counted(15)) / reps
        out(kernel=f"allreduce + residual + rmsnorm ({name})", ranks=world, rows=m_rows, d=d, us=round(ms * 1e3, 2),
            nccl_allreduce_plus_norm_us=round(ms_n * 1e3, 2))
    torch.cuda.synchronize()
    ops.check_status()
    from .runtime import finish
    finish(hard=(__name__ == "__main__"))
    return 0


if __name__ == "__main__":
    sys.exit(main())

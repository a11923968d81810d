"""Worker for the multi-GPU tests of the fused communication kernels (torch.distributed.run, one rank per GPU).

Against NCCL collectives computed by the same ranks:
  * reduce-scatter by pull into an fp32 shard, with plain peer loads and (where the symmetric buffer has an NVLink
    multicast mapping) with multimem.ld_reduce;
  * the decode all-reduce fused with the split-K reduction, the residual add and the RMS-norm, both ways, called
    many times in a row on alternating buffers;
  * two tensor-parallel decoders built one after the other on the same ranks (they share the group's signal pads and
    epoch counters), each compared with the NCCL-all-reduce decoder on the same weights and prompts.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def reduce_scatter_case(dev, rank, world):
    from cosmos_b200.parallel.symm import symm_group

    sg = symm_group(dist.group.WORLD, list(range(world)), dev)
    n = 1 << 20
    buf = sg.alloc("test_rs", n * 2)
    mine = buf.view(0, (n,), torch.bfloat16)
    ptrs = torch.tensor(buf.peer_ptrs, dtype=torch.int64, device=dev)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    x = torch.randn(n, generator=g, device=dev).bfloat16()
    mine.copy_(x)
    want_full = x.float().clone()
    dist.all_reduce(want_full)
    ns = n // world
    want = want_full[rank * ns:(rank + 1) * ns] / world
    worst = {}
    modes = [("p2p", 0)]
    mc = sg.use_multicast(buf)
    if mc:
        modes.append(("multimem", mc))
    for name, mcp in modes:
        out = torch.zeros(ns, dtype=torch.float32, device=dev)
        sq = torch.zeros(1, dtype=torch.float32, device=dev)
        sg.barrier(slot=3)
        torch.ops.cosmos_b200.reduce_scatter_pull(ptrs, mcp, world, rank * ns, out, False, 1.0 / world, sq)
        torch.ops.cosmos_b200.reduce_scatter_pull(ptrs, mcp, world, rank * ns, out, True, 1.0 / world, None)
        sg.barrier(slot=3)
        torch.cuda.synchronize()
        err = ((out - 2 * want).abs() / (1 + want.abs())).max().item()
        sq_err = abs(sq.item() - want.pow(2).sum().item()) / want.pow(2).sum().item()
        worst[name] = max(err, sq_err)
    return worst, bool(mc)


def allreduce_norm_case(dev, rank, world):
    from cosmos_b200.config import tiny128_config
    from cosmos_b200.parallel.tp import TPContext

    cfg = tiny128_config(n_heads=8, n_kv_heads=8, ffn_dim=1024)
    worst = 0.0
    for nvls in ("1", "0"):
        os.environ["COSMOS_NVLS"] = nvls
        ctx = TPContext(cfg, dist.group.WORLD, list(range(world)), dev, fused=True, sequence_parallel=False)
        for (m, n, k) in ((32, 4096, 512), (5, 1024, 4096), (200, 512, 256)):
            g = torch.Generator(device=dev).manual_seed(100 * rank + m)
            w = (torch.randn(n, k, generator=g, device=dev) / k ** 0.5).bfloat16()
            gamma = (1 + 0.1 * torch.randn(n, generator=torch.Generator(device=dev).manual_seed(5), device=dev)).bfloat16()
            ctx.begin_step()
            for it in range(6):
                a = torch.randn(m, k, generator=g, device=dev).bfloat16()
                resid = torch.randn(m, n, generator=torch.Generator(device=dev).manual_seed(it), device=dev).bfloat16()
                h, x_new = ctx.gemm_allreduce_norm(a, w, resid, gamma, 1e-6)
                y = a.float() @ w.float().t()
                dist.all_reduce(y)
                want_x = y + resid.float()
                want_h = want_x * torch.rsqrt(want_x.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
                worst = max(worst, ((x_new.float() - want_x).abs() / (1 + want_x.abs())).max().item(),
                            ((h.float() - want_h).abs() / (1 + want_h.abs())).max().item())
        torch.cuda.synchronize()
    os.environ["COSMOS_NVLS"] = "1"
    return worst


def decoder_case(dev, rank, world):
    from cosmos_b200.config import tiny128_config
    from cosmos_b200.serve.decoder import TPDecoder

    cfg = tiny128_config(n_layers=2, n_heads=8, n_kv_heads=4, ffn_dim=1024, max_text_len=64)
    first, later = {}, {}
    for name, fused in (("nccl", False), ("fused_a", True), ("fused_b", True)):
        dec = TPDecoder(cfg, world, rank, dist.group.WORLD, dev, page_size=16, max_batch=4, max_len=200, seed=3,
                        fused=fused)
        dec.prefill_synthetic(4, 64, 40, seed=11)
        dec.step()                      # same tokens and cache for every decoder: the logits must agree
        first[name] = dec.last_logits.clone()
        if fused:
            dec.capture(warmup=2)       # the captured step replays the fused collectives with device-side epochs
        out = []
        for _ in range(4):
            out.append(dec.step().clone())
        torch.cuda.synchronize()
        later[name] = (torch.stack(out), dec.last_logits.clone())
    ref = first["nccl"]
    worst = max((first[n] - ref).abs().max().item() / (1 + ref.abs().max().item()) for n in ("fused_a", "fused_b"))
    # greedy decoding of a random-weight model amplifies rounding differences, so the later steps are compared
    # between the two fused decoders only (same arithmetic, different epoch history)
    ta, la = later["fused_a"]
    tb, lb = later["fused_b"]
    ok = bool(torch.isfinite(la).all()) and bool((ta == tb).all()) and (la - lb).abs().max().item() < 1e-2 * (1 + la.abs().max().item())
    return ok, worst


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from cosmos_b200 import ops
    ops.load_extension()
    ok = True
    worst, has_mc = reduce_scatter_case(dev, rank, world)
    good = all(v < 2e-2 for v in worst.values())
    ok &= good
    if rank == 0:
        print(f"reduce-scatter pull vs NCCL: {worst} multicast mapping: {has_mc} {'OK' if good else 'MISMATCH'}", flush=True)
    ops.check_status()
    w = allreduce_norm_case(dev, rank, world)
    good = w < 3e-2
    ok &= good
    if rank == 0:
        print(f"fused all-reduce + residual + RMS-norm vs NCCL: max rel diff {w:.3g} {'OK' if good else 'MISMATCH'}", flush=True)
    ops.check_status()
    same, w = decoder_case(dev, rank, world)
    good = same and w < 5e-2
    ok &= good
    if rank == 0:
        print(f"two fused decoders in turn vs NCCL decoder: logits rel diff {w:.3g}, tokens agree: {same} "
              f"{'OK' if good else 'MISMATCH'}", flush=True)
    ops.check_status()
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() > 0 else 1)


if __name__ == "__main__":
    main()

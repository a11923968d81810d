"""Worker for the multi-GPU training test (torch.distributed.run, one rank per GPU): two FSDP
steps of a small head_dim-128 bf16 model with the fused paths (parameter gathers prefetched on a side
stream by the pull kernel, per-layer reduce-scatter by pull during backward, AdamW kernel on the fp32
gradient shards) against the NCCL-collective baseline, plus the one-shot all-reduce kernel against NCCL
all_reduce. Both paths run the forward and backward on this package's kernels (bf16 parameters) and
differ only in the collectives and the optimizer kernel."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def fsdp_case(fused):
    from cosmos_b200.config import ParallelConfig, tiny128_config
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.train import TrainConfig, Trainer

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    cfg = tiny128_config(max_text_len=32, n_layers=2)
    model = MoTModel(cfg, dtype=torch.bfloat16, device=dev, pad_to=128 * world)
    model.init_weights(seed=3)
    mesh = Mesh(ParallelConfig(dp_shard=world), world, rank)
    tr = Trainer(model, mesh, TrainConfig(lr=1e-3, max_grad_norm=0.5, fused=fused))
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    logs = []
    for _ in range(2):
        lat = torch.randn(1, 16, 3, 16, 16, generator=g, device=dev, dtype=torch.bfloat16)
        ids = torch.randint(0, cfg.vocab_size, (1, 32), generator=g, device=dev)
        t = torch.rand(1, generator=g, device=dev)
        eps = torch.randn(lat.shape, generator=g, device=dev, dtype=torch.bfloat16)
        logs.append(tr.train_step(lat, ids, t=t, eps=eps))
    torch.cuda.synchronize()
    from cosmos_b200 import ops
    ops.check_status()
    full = tr.fsdp.full_state()
    return full, logs


def allreduce_case():
    from cosmos_b200.config import tiny128_config
    from cosmos_b200.parallel.tp import TPContext

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    cfg = tiny128_config(n_heads=8, n_kv_heads=8, ffn_dim=1024)
    ctx = TPContext(cfg, dist.group.WORLD, list(range(world)), dev, fused=True, sequence_parallel=False)
    worst = 0.0
    for n in (4096, 32 * 4096):
        for it in range(3):
            x = torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(rank * 10 + it)).bfloat16()
            got = ctx._all_reduce(x.clone())
            want = x.float().clone()
            dist.all_reduce(want)
            worst = max(worst, ((got.float() - want).abs() / (1 + want.abs())).max().item())
    torch.cuda.synchronize()
    return worst


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ok = True
    base, logs_b = fsdp_case(False)
    fused, logs_f = fsdp_case(True)
    worst = max((fused[k].float() - base[k].float()).abs().max().item() for k in base)
    good = worst < 2e-2 and abs(logs_b[-1]["loss"] - logs_f[-1]["loss"]) < 2e-2
    ok &= good
    if dist.get_rank() == 0:
        print(f"fsdp fused vs baseline: max param diff {worst:.3g}, loss {logs_f[-1]['loss']:.4f} vs "
              f"{logs_b[-1]['loss']:.4f}, grad norm {logs_f[-1]['grad_norm']:.4f} vs {logs_b[-1]['grad_norm']:.4f} "
              f"{'OK' if good else 'MISMATCH'}", flush=True)
    w = allreduce_case()
    good = w < 2e-2
    ok &= good
    if dist.get_rank() == 0:
        print(f"one-shot all-reduce vs NCCL: max rel diff {w:.3g} {'OK' if good else 'MISMATCH'}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

"""Worker for the multi-GPU tests (launched with torch.distributed.run, one rank per GPU).

Runs the Generator on a small head_dim-128 model with the fused P2P paths (Ulysses all-to-all in
the QKV / attention epilogues, CFG-parallel peer loads in the sampler kernel) and checks the
result against the NCCL-collective baseline of the same layout computed by the same ranks.
NVLS is not needed: the kernels use plain peer loads and stores.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(pc_kw, steps=2):
    from cosmos_b200 import ops
    from cosmos_b200.config import ParallelConfig, SamplingConfig, tiny128_config
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.parallel.runtime import build_engine_for_mesh
    from cosmos_b200.pipeline import Cosmos3OmniPipeline

    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    cfg = tiny128_config(max_text_len=64, n_heads=8, n_kv_heads=4)
    model = MoTModel(cfg, dtype=torch.bfloat16, device=dev)
    model.init_weights(seed=5)
    presliced = bool(pc_kw.pop("presliced", False))
    mesh = Mesh(ParallelConfig(**pc_kw), world, rank)
    local = None
    if presliced:
        # the same weights as rank-local slices: a model built from the tensor-parallel local configuration
        from cosmos_b200.parallel.tp import shard_full_model, tp_local_config
        local = MoTModel(tp_local_config(cfg, mesh.size("tp")), dtype=torch.bfloat16, device=dev)
        shard_full_model(model, local, cfg, mesh.size("tp"), mesh.index("tp"))
    outs = {}
    for fused in (False, True):
        if presliced and fused:
            eng = build_engine_for_mesh(local, mesh, fused=True, full_cfg=cfg)
        else:
            eng = build_engine_for_mesh(model, mesh, fused=fused)
        g = torch.Generator(device=dev).manual_seed(1)
        ids_c = torch.randint(0, cfg.vocab_size, (1, 64), generator=g, device=dev)
        ids_u = torch.randint(0, cfg.vocab_size, (1, 64), generator=g, device=dev)
        st = eng.make_state(ids_c, ids_u, (5, 32, 32))
        sc = SamplingConfig(num_steps=steps, guidance=5.0, shift=3.0, seed=2)
        pipe = Cosmos3OmniPipeline(eng.model, None, None, None, engine=eng)
        x = pipe.begin(st, sc)
        for i in range(steps):
            x = pipe.step(x, i)
        outs[fused] = pipe.gather_tokens(x, st).float()
        torch.cuda.synchronize()
        ops.check_status()
    err = (outs[True] - outs[False]).abs().max().item()
    scale = outs[False].abs().max().item()
    return err, scale


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    layouts = json.loads(sys.argv[1]) if len(sys.argv) > 1 else [{"cp": world}]
    ok = True
    for pc in layouts:
        err, scale = run(pc)
        good = err <= 0.03 * max(scale, 1.0)
        ok = ok and good
        if dist.get_rank() == 0:
            print(f"layout {pc}: fused vs NCCL baseline max|diff| = {err:.4g} (scale {scale:.3g}) "
                  f"{'OK' if good else 'MISMATCH'}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()

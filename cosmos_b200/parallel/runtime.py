"""Process bootstrap and engine construction for a mesh.

`init_distributed` reads the torchrun environment (MASTER_ADDR, MASTER_PORT, RANK, WORLD_SIZE,
LOCAL_RANK; reference cookbooks/cosmos3/reasoner/README.md:41-42), starts NCCL (GPU) or gloo
(CPU) and builds the mesh from explicit degrees or a preset (`latency` / `throughput`).
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..config import ParallelConfig, preset_parallelism
from .mesh import Mesh


def init_distributed(world: Optional[int] = None, rank: Optional[int] = None, local_rank: Optional[int] = None,
                     preset: Optional[str] = "latency", pc: Optional[ParallelConfig] = None,
                     backend: Optional[str] = None, n_kv_heads: int = 8, use_cfg: bool = True,
                     timeout_s: int = 600) -> Mesh:
    world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    local_rank = int(os.environ.get("LOCAL_RANK", "0")) if local_rank is None else local_rank
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    if pc is None:
        pc = preset_parallelism(preset or "latency", world, use_cfg=use_cfg, n_kv_heads=n_kv_heads)
    return Mesh(pc, world, rank)


def finish(hard: bool = True, grace_s: float = 0.0) -> None:
    """End of a launcher-run entry point: the ranks synchronise their devices, meet at a barrier (after it no rank
    has a kernel or collective in flight that reads a peer's buffers), flush and leave.
    With `hard` the process then exits through `os._exit`: a communicator whose collectives were captured in a CUDA
    graph can block in `destroy_process_group`, and a rank that blocks there keeps the launcher and the GPUs busy
    long after the work is done. `grace_s > 0` first attempts the regular teardown in a helper thread for at most
    that long. Without `hard` (in-process callers such as tests) the communicators are destroyed normally."""
    import sys
    import threading

    active = dist.is_available() and dist.is_initialized()
    if active:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier()
        if not hard:
            dist.destroy_process_group()
            return
        if grace_s > 0:
            t = threading.Thread(target=dist.destroy_process_group, daemon=True)
            t.start()
            t.join(grace_s)
    sys.stdout.flush()
    sys.stderr.flush()
    if hard and active:
        os._exit(0)


def build_engine_for_mesh(model, mesh: Mesh, fused: bool = True, full_cfg=None):
    """GeneratorEngine whose attention context and CFG handling match the mesh. `full_cfg`: the full model's
    configuration when `model` was built from `parallel.tp.tp_local_config` (it holds this rank's weight slices)."""
    from ..models.generator import GeneratorEngine

    ctx = None
    cfg_group = None
    if mesh.size("cp") > 1 and mesh.size("tp") > 1:
        raise ValueError("use either context parallelism or tensor parallelism (whose head split is the Ulysses layout)")
    if mesh.size("cp") > 1:
        from .ulysses import make_cp_context
        ctx = make_cp_context(model.cfg, mesh, fused=fused)
    if mesh.size("tp") > 1:
        from .tp import TPContext
        dev = next(model.parameters()).device
        ctx = TPContext(full_cfg or model.cfg, mesh.group("tp"), mesh.group_ranks["tp"], dev, fused=fused,
                        presliced=full_cfg is not None)
    if mesh.size("cfgp") > 1:
        from .cfgp import CFGParallel
        cfg_group = CFGParallel(mesh, fused=fused)
    return GeneratorEngine(model, ctx=ctx, cfg_group=cfg_group)

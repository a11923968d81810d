"""Generator post-training: flow-matching loss on the DM tower with FSDP x context parallelism,
activation checkpointing on every block, AdamW and global-norm gradient clipping.

    torchrun --nproc-per-node 8 -m cosmos_b200.train --model Cosmos3-Nano --dp-shard-size 4 --cp-size 2 \
        --steps 10 --latent 16,16,44,80 --text-len 256

(The reference only points to a training guide in its framework repository, reference
README.md:653-655; the recipe here is: t ~ logit-normal(0, 1), x_t = (1 - t) x0 + t eps, target
v = eps - x0, MSE on the DM tokens; the AR tower provides the prompt's K/V and is frozen unless
`--train-ar` selects joint training of both towers through the block-masked attention.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .config import MoTConfig, ParallelConfig, get_model_config
from .models import rope, sampler as samplers
from .models.mot import LOCAL_ATTN, MoTModel, patchify
from .parallel.fsdp import FSDP
from .parallel.mesh import Mesh


@dataclass
class TrainConfig:
    lr: float = 1e-4
    weight_decay: float = 0.0
    max_grad_norm: Optional[float] = 1.0
    checkpoint_blocks: bool = True
    train_ar: bool = False
    t_mean: float = 0.0
    t_std: float = 1.0
    fused: bool = True
    # seconds a rank waits on the host for its peers before a step; None = no liveness protocol
    # (parallel/health.py: bounded per-step rendezvous + heartbeats over the c10d store)
    health_timeout_s: Optional[float] = None
    # optimizer steps see the mean gradient of `grad_accum` consecutive micro-batches
    grad_accum: int = 1
    # learning-rate schedule: linear warm-up over `warmup_steps`, then cosine decay to `min_lr_ratio * lr` at
    # `total_steps` (0 = constant after the warm-up)
    warmup_steps: int = 0
    total_steps: int = 0
    min_lr_ratio: float = 0.1

    def lr_at(self, step: int) -> float:
        """Learning rate of optimizer step `step` (1-based)."""
        import math
        if self.warmup_steps > 0 and step <= self.warmup_steps:
            return self.lr * step / self.warmup_steps
        if self.total_steps <= 0:
            return self.lr
        span = max(1, self.total_steps - self.warmup_steps)
        frac = min(1.0, max(0.0, (step - self.warmup_steps) / span))
        return self.lr * (self.min_lr_ratio + (1.0 - self.min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * frac)))


class Trainer:
    def __init__(self, model: MoTModel, mesh: Mesh, tc: TrainConfig):
        self.model, self.mesh, self.tc = model, mesh, tc
        self.cfg: MoTConfig = model.cfg
        dev = next(model.parameters()).device
        self.device = dev
        # parameters are sharded across the union of the dp_shard and cp axes
        ranks, group = _flat_group(mesh, ("dp_shard", "cp"))
        towers = ("ar", "dm") if tc.train_ar else ("dm",)
        if not tc.train_ar and model.has_ar:
            for n, p in model.named_parameters():
                if n.startswith("ar.") or n in ("embed", "ar_norm", "lm_head"):
                    p.requires_grad_(False)
        # replicas (dp_replicate axis) hold the same shards; their gradients are averaged at the optimizer step
        rep = mesh.size("dp_replicate")
        rep_group = mesh.group("dp_replicate") if rep > 1 and dist.is_initialized() else None
        self.fsdp = FSDP(model, group, ranks, towers, tc.fused, tc.lr, weight_decay=tc.weight_decay,
                         max_grad_norm=tc.max_grad_norm, replicate_group=rep_group, replicate_size=rep)
        self.ctx = LOCAL_ATTN
        if mesh.size("cp") > 1:
            from .parallel.ulysses import UlyssesAttn
            self.ctx = UlyssesAttn(self.cfg, mesh.group("cp"), mesh.group_ranks["cp"], dev, fused=False)
        self.cp, self.cp_rank = mesh.size("cp"), mesh.index("cp")
        self.hb = None
        if tc.health_timeout_s is not None and mesh.world > 1 and dist.is_initialized():
            from torch.distributed.distributed_c10d import _get_default_store

            from .parallel.health import Heartbeat
            self.hb = Heartbeat(_get_default_store(), mesh.rank, mesh.world)

    def loss(self, latents: torch.Tensor, text_ids: torch.Tensor, generator: Optional[torch.Generator] = None,
             t: Optional[torch.Tensor] = None, eps: Optional[torch.Tensor] = None) -> torch.Tensor:
        """latents [B, C, T, H, W] (clean), text_ids [B, n]. Every cp rank passes the SAME batch; each
        keeps its shard of the DM tokens."""
        cfg, m = self.cfg, self.model
        b = latents.shape[0]
        dev = latents.device
        if t is None:
            t = samplers.logit_normal_t(b, self.tc.t_mean, self.tc.t_std, generator, dev)
        if eps is None:
            eps = torch.randn(latents.shape, generator=generator, device=dev, dtype=latents.dtype)
        tt = t.view(b, 1, 1, 1, 1).to(latents.dtype)
        x_t = (1 - tt) * latents + tt * eps
        target = patchify(eps - latents, cfg)
        tokens = patchify(x_t, cfg)
        grid = (latents.shape[2] // cfg.patch_t, latents.shape[3] // cfg.patch_hw, latents.shape[4] // cfg.patch_hw)
        n_text = text_ids.shape[1]
        pos = rope.generator_positions(n_text, grid, device=dev)
        p_vid = pos["video"]
        s = tokens.shape[1]
        if self.cp > 1:
            assert s % self.cp == 0, "token count must be divisible by cp"
            sl = slice(self.cp_rank * (s // self.cp), (self.cp_rank + 1) * (s // self.cp))
            tokens, target, p_vid = tokens[:, sl], target[:, sl], p_vid[:, sl]
        mdt = m.patch_in.dtype
        x = m.dm_embed(tokens.to(mdt))
        if self.tc.train_ar:
            xa = m.embed_tokens(text_ids)
            _, h = m.joint_forward(xa, pos["text"], x, t, p_vid, self.ctx, self.fsdp.layer_params,
                                   self.tc.checkpoint_blocks)
        else:
            with torch.no_grad():
                _, kvs = m.ar_forward(m.embed_tokens(text_ids), pos["text"])
            h = m.dm_forward(x, t, p_vid, kvs, self.ctx, self.fsdp.layer_params, self.tc.checkpoint_blocks)
        pred = m.dm_heads(h, h.shape[1])["video"]
        return F.mse_loss(pred.float(), target.float())

    def train_step(self, latents, text_ids, generator=None, **kw) -> Dict[str, float]:
        """One optimizer step. With `health_timeout_s` the step starts only after every rank has shown up
        for it on the host (PeerFailure otherwise), and a failure of this rank is announced to the others."""
        if self.hb is not None:
            from .parallel.health import guarded_step
            return guarded_step(self.hb, lambda: self._train_step(latents, text_ids, generator, **kw),
                                self.tc.health_timeout_s)
        return self._train_step(latents, text_ids, generator, **kw)

    def _train_step(self, latents, text_ids, generator=None, **kw) -> Dict[str, float]:
        """One micro-batch: forward, backward and, on every `grad_accum`-th call, the optimizer step. The returned
        record carries `grad_norm` and `lr` only for calls that stepped."""
        from .utils.obs import nvtx_range
        acc = max(1, self.tc.grad_accum)
        with nvtx_range("train/forward"):
            loss = self.loss(latents, text_ids, generator, **kw)
        with nvtx_range("train/backward"):
            (loss / acc if acc > 1 else loss).backward()
        self._micro = getattr(self, "_micro", 0) + 1
        out: Dict[str, float] = {}
        if self._micro % acc == 0:
            with nvtx_range("train/optimizer"):
                self.fsdp.lr = self.tc.lr_at(self.fsdp.step_count + 1)
                out["grad_norm"] = self.fsdp.step()
                out["lr"] = self.fsdp.lr
        lv = loss.detach().float()
        if self.mesh.world > 1 and dist.is_initialized():
            dist.all_reduce(lv)
            lv /= self.mesh.world
        return {"loss": float(lv), **out}

    # ------------------------------------------------------------------ checkpoint / resume
    def save(self, out_dir, step: int) -> None:
        from .ckpt import safetensors_io as sio
        out = Path(out_dir)
        sio.save_train_state(out / f"train_state_rank{self.mesh.rank:05d}.safetensors", step,
                             self.fsdp.state_tensors(), {"world": self.mesh.world})

    def load(self, out_dir) -> int:
        from .ckpt import safetensors_io as sio
        step, tensors, extra = sio.load_train_state(Path(out_dir) / f"train_state_rank{self.mesh.rank:05d}.safetensors")
        if extra.get("world") != self.mesh.world:
            raise ValueError("training state was saved with a different world size")
        self.fsdp.load_state_tensors(tensors, step)
        return step


_FLAT_GROUPS: Dict[Tuple, object] = {}


def _flat_group(mesh: Mesh, axes: Tuple[str, ...]):
    """Process group over the product of several mesh axes (same other coordinates)."""
    def members(rank):
        c = mesh.coords_of(rank)
        out = []
        def rec(i, cc):
            if i == len(axes):
                out.append(mesh.rank_of(cc)); return
            for v in range(mesh.sizes[axes[i]]):
                rec(i + 1, {**cc, axes[i]: v})
        rec(0, c)
        return tuple(sorted(out))
    mine = members(mesh.rank)
    if len(mine) == 1 or not dist.is_initialized():
        return list(mine), None
    key = (axes, mesh.world)
    if key not in _FLAT_GROUPS:
        groups = {}
        for r in range(mesh.world):
            mem = members(r)
            if mem not in groups:
                groups[mem] = dist.new_group(list(mem))
        _FLAT_GROUPS[key] = groups
    return list(mine), _FLAT_GROUPS[key][mine]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--dp-shard-size", type=int, default=None)
    ap.add_argument("--dp-replicate-size", type=int, default=1)
    ap.add_argument("--cp-size", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--latent", default="16,5,16,16", help="C,T,H,W of the latent clip")
    ap.add_argument("--text-len", type=int, default=64)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--grad-accum", type=int, default=1, help="micro-batches per optimizer step")
    ap.add_argument("--lr-warmup-steps", type=int, default=0)
    ap.add_argument("--lr-total-steps", type=int, default=0, help="cosine decay to --min-lr-ratio x lr at this step (0 = constant)")
    ap.add_argument("--min-lr-ratio", type=float, default=0.1)
    ap.add_argument("--no-checkpoint", action="store_true")
    ap.add_argument("--train-ar", action="store_true")
    ap.add_argument("--save-dir", default=None)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--data-root", default=None,
                    help="folder of captioned clips (data/video_text.py); without it the step runs on synthetic latents")
    ap.add_argument("--data-fps", type=float, default=None, help="resample clips to this frame rate")
    ap.add_argument("--data-workers", type=int, default=2, help="host threads that decode and resize ahead of the GPU")
    ap.add_argument("--data-seed", type=int, default=0)
    ap.add_argument("--vae-widths", default="32,64,128,128", help="channel widths of the tokenizer VAE (with --data-root)")
    ap.add_argument("--log-jsonl", default=None, help="append one JSON record per step to this file (rank 0)")
    ap.add_argument("--health-timeout", type=float, default=None,
                    help="seconds to wait on the host for every rank before each step (peer failure detection)")
    args = ap.parse_args(argv)
    from .parallel.runtime import init_distributed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    dshard = args.dp_shard_size or world // (args.cp_size * args.dp_replicate_size)
    pc = ParallelConfig(dp_replicate=args.dp_replicate_size, dp_shard=dshard, cp=args.cp_size)
    mesh = init_distributed(world, rank, local, pc=pc)
    over = {"n_layers": args.layers} if args.layers else {}
    cfg = get_model_config(args.model, **over)
    dtype = torch.bfloat16 if cuda else torch.float32
    shard_ws = dshard * args.cp_size
    model = MoTModel(cfg, dtype=dtype, device=dev, pad_to=128 * shard_ws)
    model.init_weights(seed=0)
    tr = Trainer(model, mesh, TrainConfig(lr=args.lr, checkpoint_blocks=not args.no_checkpoint, train_ar=args.train_ar,
                                         health_timeout_s=args.health_timeout, grad_accum=args.grad_accum,
                                         warmup_steps=args.lr_warmup_steps, total_steps=args.lr_total_steps,
                                         min_lr_ratio=args.min_lr_ratio))
    step0 = tr.load(args.save_dir) if (args.resume and args.save_dir) else 0
    c, t, h, w = (int(v) for v in args.latent.split(","))
    # ranks of one cp group see the same clip; different dp ranks see different clips
    data_rank = mesh.index("dp_replicate") * mesh.size("dp_shard") + mesh.index("dp_shard")
    data_world = mesh.size("dp_replicate") * mesh.size("dp_shard")
    feed = batcher = None
    if args.data_root:
        from .data.video_text import LatentBatcher, Prefetcher, ShardedSampler, VideoTextDataset
        from .models.vae import CausalVideoVAE
        from .utils.tokenizer import load_tokenizer
        ds = VideoTextDataset(args.data_root, 1 + (t - 1) * cfg.vae_t_compress, w * cfg.vae_s_compress,
                              h * cfg.vae_s_compress, args.data_fps)
        sampler = ShardedSampler(len(ds), data_rank, data_world, args.data_seed)
        state_file = Path(args.save_dir) / f"data_state_rank{rank:05d}.json" if args.save_dir else None
        if args.resume and state_file is not None and state_file.exists():
            sampler.load_state_dict(json.loads(state_file.read_text()))
        vae = CausalVideoVAE(c, tuple(int(v) for v in args.vae_widths.split(","))).to(device=dev, dtype=dtype).eval()
        batcher = LatentBatcher(vae, load_tokenizer(None, cfg.vocab_size), args.text_len, cfg.vocab_size, dev, dtype)
        feed = Prefetcher(ds, sampler, args.micro_batch, depth=2, workers=args.data_workers)
    g = torch.Generator(device=dev).manual_seed(1000 + data_rank)
    tokens_per_step = args.micro_batch * (t // cfg.patch_t) * (h // cfg.patch_hw) * (w // cfg.patch_hw)
    tokens_per_step = (tokens_per_step + args.micro_batch * args.text_len) * mesh.size("dp_shard") * mesh.size("dp_replicate")
    from .utils.obs import JsonlLogger
    logger = JsonlLogger(args.log_jsonl, stdout=True)  # rank 0 only
    times = []
    for s in range(step0, step0 + args.warmup + args.steps):
        if feed is not None:
            lat, ids = batcher(next(feed))
        else:
            lat = torch.randn(args.micro_batch, c, t, h, w, generator=g, device=dev, dtype=dtype)
            ids = torch.randint(0, cfg.vocab_size, (args.micro_batch, args.text_len), generator=g, device=dev)
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = tr.train_step(lat, ids, g)
        if cuda:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if s >= step0 + args.warmup:
            times.append(dt)
        logger.log(step=s + 1, **out, step_s=round(dt, 4))
    if args.save_dir:
        tr.save(args.save_dir, step0 + args.warmup + args.steps)
        if feed is not None:   # where the data stream of this rank continues after a resume
            state_file.write_text(json.dumps(feed.resume_state))
    if feed is not None:
        feed.close()
    if rank == 0 and times:
        avg = sum(times) / len(times)
        print(json.dumps({"metric": "train_tokens_per_s", "value": tokens_per_step / avg, "step_s": avg,
                          "tokens_per_step": tokens_per_step, "parallelism": mesh.describe(), "model": cfg.name}))
    if world > 1:
        from .parallel.runtime import finish
        finish(hard=(__name__ == "__main__"))
    return 0


if __name__ == "__main__":
    sys.exit(main())

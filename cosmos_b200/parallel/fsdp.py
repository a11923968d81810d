"""Fully-sharded data parallelism (ZeRO-3 style) over the model's per-layer flat parameters.

Every `FlatLayer.flat` is split evenly across the shard group; a rank keeps only its slice
(bf16/fp32 parameter shard, fp32 master copy, AdamW moments). A layer's full parameters exist
only while the layer runs:

  forward / recompute : all-gather the shards (autograd function `_Gather`)
  backward            : reduce-scatter the full gradient back to shard owners

Baseline path (any device, CPU/gloo included): `all_gather_into_tensor` / `reduce_scatter_tensor`.
Fused path (CUDA): shards live in symmetric memory; the gather is ONE pull kernel that reads all
peers' shards over NVLink at once (`allgather_pull`), and the reduce-scatter is folded into the
optimizer: full bf16 gradients stay in a symmetric buffer and the shard owner's
`rs_adamw` kernel pulls the matching slices from every peer, reduces them in fp32 and applies
AdamW (+ global-norm clipping via a two-pass variant) without a collective call or an
intermediate reduced-gradient tensor in bf16.

Parameters outside the layers (embeddings, patch/time projections, heads) are replicated and
their gradients all-reduced; they are a small part of the DM tower.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.mot import FlatLayer, MoTModel
from .symm import SymmGroup, symm_group


class _Gather(torch.autograd.Function):
    """shard [n/ws] -> full [n]; backward reduce-scatters (mean over the group is applied by the
    caller through the loss scaling, here gradients are summed)."""

    @staticmethod
    def forward(ctx, shard: torch.Tensor, unit: "ShardedUnit"):
        ctx.unit = unit
        return unit.gather()

    @staticmethod
    def backward(ctx, grad_full: torch.Tensor):
        return ctx.unit.scatter_grad(grad_full), None


class ShardedUnit:
    """One flat parameter tensor sharded across the group."""

    def __init__(self, layer: FlatLayer, group, ws: int, rank: int, sg: Optional[SymmGroup], name: str):
        self.layer, self.group, self.ws, self.rank, self.sg, self.name = layer, group, ws, rank, sg, name
        full = layer.flat.data
        n = full.numel()
        assert n % ws == 0, "flat parameter length must be divisible by the shard count (use pad_to)"
        self.n, self.ns = n, n // ws
        self.dtype, self.device = full.dtype, full.device
        shard = full[rank * self.ns:(rank + 1) * self.ns].clone()
        self.fused = sg is not None
        if self.fused:
            es = full.element_size()
            buf = sg.alloc(f"fsdp_shard_{name}", self.ns * es)
            self.shard_store = buf.view(0, (self.ns,), self.dtype)
            self.shard_store.copy_(shard)
            self.shard_ptrs = torch.tensor([buf.peer_addr(r) for r in range(ws)], dtype=torch.int64, device=self.device)
            self.shard = nn.Parameter(self.shard_store)
        else:
            self.shard = nn.Parameter(shard)
        # free the replicated full tensor
        layer.flat = nn.Parameter(torch.empty(0, dtype=self.dtype, device=self.device), requires_grad=False)
        self.master = self.shard.data.float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_full: Optional[torch.Tensor] = None  # fused path: full bf16 grads in symmetric memory

    def gather(self) -> torch.Tensor:
        full = torch.empty(self.n, dtype=self.dtype, device=self.device)
        if self.ws == 1:
            full.copy_(self.shard.data)
        elif self.fused:
            torch.ops.cosmos_b200.allgather_pull(self.shard_ptrs, self.ws, full, self.ns * full.element_size())
        else:
            dist.all_gather_into_tensor(full, self.shard.data.contiguous(), group=self.group)
        return full

    def scatter_grad(self, grad_full: torch.Tensor) -> torch.Tensor:
        if self.ws == 1:
            return grad_full
        if self.fused:
            # keep the full gradient where the peers can read it; the optimizer kernel reduces it
            if self.grad_full is None:
                buf = self.sg.alloc(f"fsdp_grad_{self.name}", self.n * grad_full.element_size())
                self.grad_full = buf.view(0, (self.n,), self.dtype)
                self.grad_ptrs = torch.tensor([buf.peer_addr(r) for r in range(self.ws)], dtype=torch.int64,
                                              device=self.device)
                self._has_grad = False
            if self._has_grad:
                self.grad_full.add_(grad_full)
            else:
                self.grad_full.copy_(grad_full)
                self._has_grad = True
            return torch.zeros_like(self.shard)
        out = torch.empty(self.ns, dtype=grad_full.dtype, device=grad_full.device)
        dist.reduce_scatter_tensor(out, grad_full.contiguous(), group=self.group)
        return out


class FSDP:
    def __init__(self, model: MoTModel, group, ranks: List[int], towers=("dm",), fused: bool = True,
                 lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: Optional[float] = 1.0):
        self.model, self.group = model, group
        self.ws = len(ranks)
        self.rank = ranks.index(dist.get_rank()) if dist.is_initialized() else 0
        dev = next(model.parameters()).device
        self.fused = bool(fused) and dev.type == "cuda" and self.ws > 1
        self.sg = symm_group(group, ranks, dev) if self.fused else None
        self.units: Dict[Tuple[str, int], ShardedUnit] = {}
        for t in towers:
            tower = getattr(model, t)
            for i, layer in enumerate(tower.layers):
                self.units[(t, i)] = ShardedUnit(layer, group, self.ws, self.rank, self.sg, f"{t}{i}")
        self.replicated = [p for n, p in model.named_parameters()
                           if p.requires_grad and p.numel() > 0 and ".layers." not in n]
        self.rep_master = [p.data.float().clone() for p in self.replicated]
        self.rep_m = [torch.zeros_like(m) for m in self.rep_master]
        self.rep_v = [torch.zeros_like(m) for m in self.rep_master]
        self.lr, self.betas, self.eps, self.wd, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.step_count = 0

    # ------------------------------------------------------------------ forward hook
    def layer_params(self, tower: str, i: int) -> Dict[str, torch.Tensor]:
        """Called by the model for every layer (and again during recompute): gathers the layer's
        parameters through the autograd function so that backward reduce-scatters the gradient."""
        unit = self.units.get((tower, i))
        layer = getattr(self.model, tower).layers[i]
        if unit is None:
            return layer.views()
        full = _Gather.apply(unit.shard, unit)
        return layer.views(full)

    def parameters(self):
        return [u.shard for u in self.units.values()] + self.replicated

    # ------------------------------------------------------------------ optimizer
    @torch.no_grad()
    def step(self) -> float:
        """Global-norm clip + AdamW on the shards (and the replicated parameters). Returns the
        gradient norm before clipping."""
        self.step_count += 1
        b1, b2 = self.betas
        ws = self.ws
        # replicated parameters: all-reduce (mean) their gradients
        for p in self.replicated:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            if ws > 1:
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(ws)
        inv_ws = 1.0 / ws
        sq = torch.zeros(1, dtype=torch.float32, device=self.replicated[0].device if self.replicated else "cpu")
        reduced: Dict[Tuple[str, int], torch.Tensor] = {}
        if self.fused:
            self.sg.barrier(slot=3)  # every rank's full gradients are in place
            for key, u in self.units.items():
                if u.grad_full is None or not u._has_grad:
                    continue
                red = torch.empty(u.ns, dtype=torch.float32, device=u.device)
                torch.ops.cosmos_b200.rs_adamw(u.grad_ptrs, ws, u.rank * u.ns, u.master, u.exp_avg, u.exp_avg_sq,
                                               u.shard.data, 1.0, 0.0, b1, b2, self.eps, 0.0, self.step_count, 1,
                                               sq, red)
                reduced[key] = red
            sq.mul_(inv_ws * inv_ws)
        elif self._local_kernel():
            # gradients are already local (one rank, or the NCCL reduce-scatter ran in backward): the same
            # optimizer kernel with this rank's gradient shard as its only source
            ptrs: Dict[Tuple[str, int], torch.Tensor] = {}
            for key, u in self.units.items():
                g = u.shard.grad
                if g is None:
                    continue
                g = g.contiguous()
                u.shard.grad = g  # keep the tensor alive until the update kernel below has read it
                ptrs[key] = torch.tensor([g.data_ptr()], dtype=torch.int64, device=u.device)
                red = torch.empty(u.ns, dtype=torch.float32, device=u.device)
                torch.ops.cosmos_b200.rs_adamw(ptrs[key], 1, 0, u.master, u.exp_avg, u.exp_avg_sq, u.shard.data, 1.0, 0.0,
                                               b1, b2, self.eps, 0.0, self.step_count, 1, sq, red)
                reduced[key] = red
            sq.mul_(inv_ws * inv_ws)
        else:
            for key, u in self.units.items():
                if u.shard.grad is not None:
                    g = u.shard.grad.float() * inv_ws
                    reduced[key] = g
                    sq += g.pow(2).sum()
        if ws > 1:
            dist.all_reduce(sq, group=self.group)
        rep_sq = sum(p.grad.float().pow(2).sum() for p in self.replicated) if self.replicated else 0.0
        total = float(torch.sqrt(sq + rep_sq))
        clip = 1.0
        if self.max_grad_norm is not None and total > self.max_grad_norm:
            clip = self.max_grad_norm / (total + 1e-6)
        bc1 = 1.0 - b1 ** self.step_count
        bc2 = 1.0 - b2 ** self.step_count
        for key, u in self.units.items():
            if key not in reduced:
                continue
            if self.fused:
                torch.ops.cosmos_b200.rs_adamw(u.grad_ptrs, ws, u.rank * u.ns, u.master, u.exp_avg, u.exp_avg_sq,
                                               u.shard.data, clip * inv_ws, self.lr, b1, b2, self.eps, self.wd,
                                               self.step_count, 2, None, reduced[key])
                u._has_grad = False
            elif self._local_kernel():
                torch.ops.cosmos_b200.rs_adamw(ptrs[key], 1, 0, u.master, u.exp_avg, u.exp_avg_sq, u.shard.data,
                                               clip * inv_ws, self.lr, b1, b2, self.eps, self.wd, self.step_count, 2,
                                               None, reduced[key])
                u.shard.grad = None
            else:
                _adamw(u.master, u.exp_avg, u.exp_avg_sq, reduced[key] * clip, self.lr, b1, b2, self.eps, self.wd,
                       bc1, bc2)
                u.shard.data.copy_(u.master)
                u.shard.grad = None
        for p, mst, m, v in zip(self.replicated, self.rep_master, self.rep_m, self.rep_v):
            _adamw(mst, m, v, p.grad.float() * clip, self.lr, b1, b2, self.eps, self.wd, bc1, bc2)
            p.data.copy_(mst)
            p.grad = None
        if self.fused:
            self.sg.barrier(slot=4)  # peers are done reading this step's gradients
        return total

    def _local_kernel(self) -> bool:
        """AdamW through the optimizer kernel on this rank's own gradient shards (no peer reads)."""
        if self.fused or not self.units:
            return False
        u = next(iter(self.units.values()))
        from .. import ops
        return u.device.type == "cuda" and u.dtype == torch.bfloat16 and ops.load_extension(build_if_missing=False)

    # ------------------------------------------------------------------ checkpointing
    def state_tensors(self) -> Dict[str, torch.Tensor]:
        out = {}
        for (t, i), u in self.units.items():
            out[f"{t}.{i}.master"] = u.master
            out[f"{t}.{i}.exp_avg"] = u.exp_avg
            out[f"{t}.{i}.exp_avg_sq"] = u.exp_avg_sq
        for j, (mst, m, v) in enumerate(zip(self.rep_master, self.rep_m, self.rep_v)):
            out[f"rep.{j}.master"], out[f"rep.{j}.exp_avg"], out[f"rep.{j}.exp_avg_sq"] = mst, m, v
        return out

    @torch.no_grad()
    def load_state_tensors(self, tensors: Dict[str, torch.Tensor], step: int) -> None:
        for k, dst in self.state_tensors().items():
            dst.copy_(tensors[k])
        for u in self.units.values():
            u.shard.data.copy_(u.master)
        for p, mst in zip(self.replicated, self.rep_master):
            p.data.copy_(mst)
        self.step_count = step

    @torch.no_grad()
    def full_state(self) -> Dict[str, torch.Tensor]:
        """Gathers every unit (for saving an unsharded model checkpoint)."""
        out = {}
        for (t, i), u in self.units.items():
            full = u.gather()
            layer = getattr(self.model, t).layers[i]
            for name, v in layer.views(full).items():
                out[f"{t}.layers.{i}.{name}"] = v.clone()
        return out


def _adamw(w, m, v, g, lr, b1, b2, eps, wd, bc1, bc2):
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    w.sub_(lr * ((m / bc1) / ((v / bc2).sqrt() + eps) + wd * w))

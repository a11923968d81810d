"""Fully-sharded data parallelism (ZeRO-3 style) over the model's per-layer flat parameters.

Every `FlatLayer.flat` is split evenly across the shard group; a rank keeps only its slice
(bf16/fp32 parameter shard, fp32 master copy, AdamW moments). A layer's full parameters exist
only while the layer runs:

  forward / recompute : all-gather the shards (autograd function `_Gather`)
  backward            : reduce-scatter the full gradient back to shard owners

Baseline path (any device, CPU/gloo included): `all_gather_into_tensor` / `reduce_scatter_tensor`.
Fused path (CUDA): shards live in symmetric memory and both collectives run on a side stream, overlapped
with the layers' compute:
  * gather: ONE pull kernel reads all peers' shards over NVLink at once (`allgather_pull`); while layer i
    computes, layer i + 1's gather (i - 1 during backward recomputation) is already in flight.
  * reduce-scatter: as soon as a layer's full gradient exists (the backward of `_Gather`), it is copied into
    one of two rotating symmetric buffers, the ranks meet on the device, and every shard owner pulls and adds
    its slice from all peers in fp32 (`reduce_scatter_pull`: 16-byte peer loads, or one `multimem.ld_reduce`
    per vector when the buffer has an NVLink multicast mapping). Only the fp32 gradient SHARD stays resident;
    the layer's full gradient is gone when its backward returns.
  * optimizer: global-norm clipping from the shards' sums of squares, then one AdamW kernel per shard
    (`adamw_shard`: fp32 master + moments, bf16 parameter shard rewritten in place in symmetric memory).

With a replicate axis (`replicate_group`), the reduced gradient shards, the replicated parameters' gradients and
the norm are averaged over it as well, so replicas stay bit-identical.

Parameters outside the layers (embeddings, patch/time projections, heads) are replicated and
their gradients all-reduced; they are a small part of the DM tower.
"""
from __future__ import annotations

import os
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

    def __init__(self, layer: FlatLayer, group, ws: int, rank: int, sg: Optional[SymmGroup], name: str,
                 owner: Optional["FSDP"] = None):
        self.layer, self.group, self.ws, self.rank, self.sg, self.name = layer, group, ws, rank, sg, name
        self.owner = owner
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
        self.grad_shard: Optional[torch.Tensor] = None  # fused path: reduced fp32 gradient of this rank's shard
        self._has_grad = False
        self._prefetched = None                         # (full tensor, event) of a gather in flight

    # ------------------------------------------------------------------ gather
    def _pull(self, full: torch.Tensor) -> None:
        torch.ops.cosmos_b200.allgather_pull(self.shard_ptrs, self.ws, full, self.ns * full.element_size())

    def prefetch(self, comm: "torch.cuda.Stream") -> None:
        """Starts this unit's gather on the side stream. The destination is allocated on the compute stream; the
        side stream first waits for the work enqueued there so far (the previous layer), so the pull overlaps
        the layer that is enqueued next."""
        if self._prefetched is not None or not self.fused or self.ws == 1:
            return
        cur = torch.cuda.current_stream()
        full = torch.empty(self.n, dtype=self.dtype, device=self.device)
        comm.wait_stream(cur)
        with torch.cuda.stream(comm):
            self._pull(full)
            ev = torch.cuda.Event()
            ev.record(comm)
        full.record_stream(comm)
        self._prefetched = (full, ev)

    def gather(self) -> torch.Tensor:
        if self._prefetched is not None:
            full, ev = self._prefetched
            self._prefetched = None
            torch.cuda.current_stream().wait_event(ev)
            return full
        full = torch.empty(self.n, dtype=self.dtype, device=self.device)
        if self.ws == 1:
            full.copy_(self.shard.data)
        elif self.fused:
            self._pull(full)
        else:
            dist.all_gather_into_tensor(full, self.shard.data.contiguous(), group=self.group)
        return full

    # ------------------------------------------------------------------ reduce-scatter
    def scatter_grad(self, grad_full: torch.Tensor):
        if self.ws == 1:
            return grad_full
        if self.fused:
            self.owner._reduce_scatter_async(self, grad_full)
            return None   # the reduced gradient lives in self.grad_shard (fp32)
        out = torch.empty(self.ns, dtype=grad_full.dtype, device=grad_full.device)
        dist.reduce_scatter_tensor(out, grad_full.contiguous(), group=self.group)
        return out


class FSDP:
    def __init__(self, model: MoTModel, group, ranks: List[int], towers=("dm",), fused: bool = True,
                 lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: Optional[float] = 1.0, replicate_group=None, replicate_size: int = 1,
                 overlap: bool = True):
        self.model, self.group = model, group
        self.ws = len(ranks)
        self.rank = ranks.index(dist.get_rank()) if dist.is_initialized() else 0
        self.rep_group, self.rep = replicate_group, max(1, int(replicate_size))
        dev = next(model.parameters()).device
        self.fused = bool(fused) and dev.type == "cuda" and self.ws > 1
        self.overlap = bool(overlap) and self.fused
        self.sg = symm_group(group, ranks, dev) if self.fused else None
        self.comm = torch.cuda.Stream(device=dev) if self.fused else None
        self.units: Dict[Tuple[str, int], ShardedUnit] = {}
        for t in towers:
            tower = getattr(model, t)
            for i, layer in enumerate(tower.layers):
                self.units[(t, i)] = ShardedUnit(layer, group, self.ws, self.rank, self.sg, f"{t}{i}", self)
        self._keys = list(self.units.keys())
        self._last_key: Optional[Tuple[str, int]] = None
        self._rs_count = 0
        self._gbufs = None
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
        if self.overlap:
            self._prefetch_neighbour((tower, i))
        return layer.views(full)

    def _prefetch_neighbour(self, key: Tuple[str, int]) -> None:
        """Starts the gather of the unit that will be asked for next: the following one while walking forward, the
        preceding one while backward recomputation walks the layers in reverse."""
        idx = self._keys.index(key)
        last = self._keys.index(self._last_key) if self._last_key in self.units else None
        self._last_key = key
        if last is not None and last == idx + 1:
            step = -1
        elif last is not None and last == idx - 1:
            step = 1
        else:
            step = 1 if idx == 0 else (-1 if idx == len(self._keys) - 1 else 0)
        nxt = idx + step
        if step and 0 <= nxt < len(self._keys):
            self.units[self._keys[nxt]].prefetch(self.comm)

    def parameters(self):
        return [u.shard for u in self.units.values()] + self.replicated

    # ------------------------------------------------------------------ reduce-scatter during backward
    def _reduce_scatter_async(self, u: ShardedUnit, grad_full: torch.Tensor) -> None:
        """Side stream: full gradient -> rotating symmetric buffer -> device barrier -> this rank pulls and adds its
        slice from every peer into the unit's fp32 gradient shard. Buffer b is rewritten two units later; by then
        this rank has passed the barrier of the unit in between, which every peer reaches only after its reads of
        buffer b, so one barrier per unit is enough."""
        if self._gbufs is None:
            nmax = max(x.n for x in self.units.values())
            self._gbufs = []
            for b in range(2):
                buf = self.sg.alloc(f"fsdp_gradbuf_{b}", nmax * 2)
                self._gbufs.append((buf.view(0, (nmax,), torch.bfloat16),
                                    torch.tensor(buf.peer_ptrs, dtype=torch.int64, device=u.device),
                                    # plain peer loads by default: measured 621 GB/s per rank against 519 with
                                    # multimem.ld_reduce on 4 GPUs (626 against 330 on 2)
                                    self.sg.use_multicast(buf) if os.environ.get("COSMOS_FSDP_NVLS") == "1" else 0))
        view, ptrs, mc = self._gbufs[self._rs_count & 1]
        self._rs_count += 1
        if u.grad_shard is None:
            u.grad_shard = torch.empty(u.ns, dtype=torch.float32, device=u.device)
        cur = torch.cuda.current_stream()
        comm = self.comm if self.overlap else cur
        g = grad_full.reshape(-1)
        if g.dtype != torch.bfloat16:
            g = g.to(torch.bfloat16)
        if comm is not cur:
            comm.wait_stream(cur)
        with torch.cuda.stream(comm):
            view[:u.n].copy_(g)
            self.sg.barrier(slot=3)
            torch.ops.cosmos_b200.reduce_scatter_pull(ptrs, mc, self.ws, u.rank * u.ns, u.grad_shard, u._has_grad,
                                                      1.0 / self.ws, None)
        if comm is not cur:
            g.record_stream(comm)
        u._has_grad = True

    # ------------------------------------------------------------------ optimizer
    def _avg_over_replicas(self, t: torch.Tensor) -> None:
        if self.rep > 1 and self.rep_group is not None:
            dist.all_reduce(t, group=self.rep_group)
            t.div_(self.rep)

    @torch.no_grad()
    def step(self) -> float:
        """Global-norm clip + AdamW on the shards (and the replicated parameters). Returns the
        gradient norm before clipping."""
        self.step_count += 1
        self._last_key = None
        for u in self.units.values():
            u._prefetched = None   # a gather that nobody consumed would hold the parameters from before this update
        b1, b2 = self.betas
        ws = self.ws
        # replicated parameters: all-reduce (mean) their gradients over the shard group and the replicas
        for p in self.replicated:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            if ws > 1:
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(ws)
            self._avg_over_replicas(p.grad)
        inv_ws = 1.0 / ws
        sq = torch.zeros(1, dtype=torch.float32, device=self.replicated[0].device if self.replicated else "cpu")
        reduced: Dict[Tuple[str, int], torch.Tensor] = {}
        if self.fused:
            if self.comm is not None:
                torch.cuda.current_stream().wait_stream(self.comm)   # every layer's reduce-scatter has been enqueued
            for key, u in self.units.items():
                if u.grad_shard is None or not u._has_grad:
                    continue
                self._avg_over_replicas(u.grad_shard)
                reduced[key] = u.grad_shard
            if reduced:
                norms = torch._foreach_norm(list(reduced.values()))
                sq += torch.stack(norms).pow(2).sum()
        elif self._local_kernel() and self.rep == 1:
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
                # pass 1 only adds up the squares; pass 2 reads the bf16 gradient again (no fp32 copy is kept)
                torch.ops.cosmos_b200.rs_adamw(ptrs[key], 1, 0, u.master, u.exp_avg, u.exp_avg_sq, u.shard.data, 1.0, 0.0,
                                               b1, b2, self.eps, 0.0, self.step_count, 1, sq, None)
                reduced[key] = g
            sq.mul_(inv_ws * inv_ws)
        else:
            for key, u in self.units.items():
                if u.shard.grad is not None:
                    g = u.shard.grad.float() * inv_ws
                    self._avg_over_replicas(g)
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
                if u.dtype == torch.bfloat16:
                    torch.ops.cosmos_b200.adamw_shard(reduced[key], u.master, u.exp_avg, u.exp_avg_sq, u.shard.data,
                                                      clip, self.lr, b1, b2, self.eps, self.wd, self.step_count)
                else:
                    _adamw(u.master, u.exp_avg, u.exp_avg_sq, reduced[key] * clip, self.lr, b1, b2, self.eps, self.wd,
                           bc1, bc2)
                    u.shard.data.copy_(u.master)
                u._has_grad = False
            elif self._local_kernel() and self.rep == 1:
                torch.ops.cosmos_b200.rs_adamw(ptrs[key], 1, 0, u.master, u.exp_avg, u.exp_avg_sq, u.shard.data,
                                               clip * inv_ws, self.lr, b1, b2, self.eps, self.wd, self.step_count, 0,
                                               None, None)
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
            self.sg.barrier(slot=4)  # every rank's shards are updated before anyone gathers them again
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

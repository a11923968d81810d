"""Ring-KV context parallelism: every rank keeps its query shard and visits the K/V shards of
all ranks one hop at a time, merging the per-hop partial attention with its log-sum-exp.
(The reference does not name a ring variant; it is the context-parallel mode for degrees that
the head counts do not divide, e.g. cp > 8 KV heads, or when heads are already split by TP.)

NVSwitch gives every pair of GPUs the same bandwidth, so "ring" is only a schedule: at hop i
rank r reads the shard of rank (r + i) mod cp. On CUDA the ranks' K/V shards live in symmetric
memory and ONE flash-attention launch per layer walks all of them: the kernel gets one tensor map per
source (the prompt prefix, this rank's shard, then the peers' shards in rank-staggered order) and keeps
the running max, the row sums and the output accumulator in registers and tensor memory across sources:
no partial outputs, no log-sum-exp merge, no concatenation copy. Where the peers' K/V come from is a
choice (`COSMOS_RING_MODE`):
  * `gather` (default): a pull kernel first copies every peer's shard into local staging buffers (each
    byte crosses NVLink once; rank-staggered, so no peer is read by everybody at once), then the attention
    kernel reads local memory only. Every (query block, head) CTA re-reads its K/V head, which the local
    L2 serves; data read straight from a peer is not cached locally.
  * `remote`: the attention kernel's TMA loads pull the peers' tiles over NVLink straight into shared
    memory. One launch and no staging, but every CTA's tile then crosses NVLink: measured 5 x slower than
    `gather` at 111,600 tokens on 4 GPUs (20.1 s against 3.8 s per guided step), so it is meant for short
    query shards only.
  * `staged`: the earlier schedule (a copy kernel on a side stream per hop + one attention launch per hop +
    an fp32 merge of the partial outputs).
On CPU (gloo) the shards are exchanged with all_gather and visited in the same order, which is the oracle
for the schedule.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..config import MoTConfig
from ..models.mot import KV, AttnContext, qkv_project_local
from .symm import symm_group


def merge_partial(o_run: Optional[torch.Tensor], lse_run: Optional[torch.Tensor], o_new: torch.Tensor,
                  lse_new: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combines two attention partials over disjoint key sets. o [B, S, H, D] (fp32 running),
    lse [B, H, S] natural log."""
    if o_run is None:
        return o_new.float(), lse_new.float()
    lse = torch.logaddexp(lse_run, lse_new)
    w_old = torch.exp(lse_run - lse).permute(0, 2, 1)[..., None]
    w_new = torch.exp(lse_new - lse).permute(0, 2, 1)[..., None]
    return o_run * w_old + o_new.float() * w_new, lse


class RingAttn(AttnContext):
    def __init__(self, cfg: MoTConfig, group, ranks: List[int], device, fused: bool = True):
        self.cfg, self.group = cfg, group
        self.cp = len(ranks)
        self.rank = ranks.index(dist.get_rank())
        self.device = torch.device(device)
        self.fused = bool(fused) and self.device.type == "cuda" and cfg.head_dim == 128
        self.sg = symm_group(group, ranks, device) if self.fused else None
        self._ws: Dict = {}
        self._side = torch.cuda.Stream() if self.fused else None
        self._prefix: Optional[KV] = None
        self._kv_local: Optional[KV] = None

    def qkv_project(self, h, w, cos, sin, q_norm, k_norm, cfg: MoTConfig, prefix: Optional[KV] = None):
        q, k, v = qkv_project_local(h, w, cos, sin, q_norm, k_norm, cfg)
        self._prefix = prefix
        return q, k.contiguous(), v.contiguous()

    # ------------------------------------------------------------------ schedules
    def _attend_gloo(self, q, k, v, mask):
        ks = [torch.empty_like(k) for _ in range(self.cp)]
        vs = [torch.empty_like(v) for _ in range(self.cp)]
        dist.all_gather(ks, k, group=self.group)
        dist.all_gather(vs, v, group=self.group)
        o_run = lse_run = None
        if self._prefix is not None:
            o, lse = ops.attention(q, self._prefix[0], self._prefix[1], mask=ops.MASK_FULL, return_lse=True)
            o_run, lse_run = merge_partial(None, None, o, lse)
        for i in range(self.cp):
            src = (self.rank + i) % self.cp
            o, lse = ops.attention(q, ks[src], vs[src], mask=ops.MASK_FULL, return_lse=True)
            o_run, lse_run = merge_partial(o_run, lse_run, o, lse)
        return o_run.to(q.dtype)

    def _buffers(self, k):
        key = tuple(k.shape)
        if key not in self._ws:
            nbytes = k.numel() * k.element_size()
            nb = (nbytes + 255) // 256 * 256
            buf = self.sg.alloc(f"ring_kv_{key}", 2 * nb)
            k_sym = buf.view(0, key, k.dtype)
            v_sym = buf.view(nb, key, k.dtype)
            k_ptrs = [buf.peer_addr(r, 0) for r in range(self.cp)]
            v_ptrs = [buf.peer_addr(r, nb) for r in range(self.cp)]
            stage = [(torch.empty_like(k), torch.empty_like(k)) for _ in range(2)]
            ptr1 = lambda a: torch.tensor([a], dtype=torch.int64, device=k.device)  # noqa: E731
            self._ws[key] = (k_sym, v_sym, [ptr1(p) for p in k_ptrs], [ptr1(p) for p in v_ptrs], stage, nbytes)
        return self._ws[key]

    def _attend_in_kernel(self, q, k, v, remote: bool):
        """One attention launch over the prefix, the own shard and the peers' shards. `remote`: the kernel's TMA loads
        read the peers' symmetric buffers directly; otherwise a pull kernel copies them into local staging first."""
        k_sym, v_sym, k_ptrs, v_ptrs, _, nbytes = self._buffers(k)
        key = ("addr", tuple(k.shape))
        if key not in self._ws:
            buf = self.sg._bufs[f"ring_kv_{tuple(k.shape)}"]
            nb = (k.numel() * k.element_size() + 255) // 256 * 256
            self._ws[key] = ([buf.peer_addr(r, 0) for r in range(self.cp)], [buf.peer_addr(r, nb) for r in range(self.cp)])
        ka, va = self._ws[key]
        k_sym.copy_(k)
        v_sym.copy_(v)
        self.sg.barrier(slot=5)  # every rank's shard is published
        order = [(self.rank + i) % self.cp for i in range(self.cp)]
        if remote:
            kp = [ka[r] for r in order]
            vp = [va[r] for r in order]
        else:
            skey = ("stage", tuple(k.shape))
            if skey not in self._ws:
                self._ws[skey] = [(torch.empty_like(k), torch.empty_like(k)) for _ in range(self.cp - 1)]
            stage = self._ws[skey]
            kp, vp = [k_sym.data_ptr()], [v_sym.data_ptr()]
            for i, r in enumerate(order[1:]):
                torch.ops.cosmos_b200.allgather_pull(k_ptrs[r], 1, stage[i][0], nbytes)
                torch.ops.cosmos_b200.allgather_pull(v_ptrs[r], 1, stage[i][1], nbytes)
                kp.append(stage[i][0].data_ptr())
                vp.append(stage[i][1].data_ptr())
        lens = [k.shape[1]] * self.cp
        if self._prefix is not None:
            pk, pv = self._prefix[0].contiguous(), self._prefix[1].contiguous()
            self._keep = (pk, pv)
            kp, vp, lens = [pk.data_ptr()] + kp, [pv.data_ptr()] + vp, [pk.shape[1]] + lens
        o = torch.ops.cosmos_b200.attn_fwd_sources(q, kp, vp, lens, k.shape[2], 1.0 / (q.shape[-1] ** 0.5), None)
        self.sg.barrier(slot=6)  # peers are done reading this layer's shards
        return o

    def _attend_fused(self, q, k, v, mask):
        import os
        mode = os.environ.get("COSMOS_RING_MODE", "staged" if os.environ.get("COSMOS_RING_STAGED") == "1" else "gather")
        if mode in ("gather", "remote") and self.cp + 1 <= 9:
            return self._attend_in_kernel(q, k, v, remote=(mode == "remote"))
        k_sym, v_sym, k_ptrs, v_ptrs, stage, nbytes = self._buffers(k)
        k_sym.copy_(k)
        v_sym.copy_(v)
        self.sg.barrier(slot=5)  # every rank's shard is published
        main = torch.cuda.current_stream()
        o_run = lse_run = None
        if self._prefix is not None:
            o, lse = ops.attention(q, self._prefix[0], self._prefix[1], mask=ops.MASK_FULL, return_lse=True)
            o_run, lse_run = merge_partial(None, None, o, lse)
        ready = [None, None]
        consumed = [None, None]

        def fetch(i):
            src = (self.rank + i) % self.cp
            slot = i & 1
            with torch.cuda.stream(self._side):
                if consumed[slot] is not None:
                    self._side.wait_event(consumed[slot])
                torch.ops.cosmos_b200.allgather_pull(k_ptrs[src], 1, stage[slot][0], nbytes)
                torch.ops.cosmos_b200.allgather_pull(v_ptrs[src], 1, stage[slot][1], nbytes)
                ev = torch.cuda.Event()
                ev.record(self._side)
                ready[slot] = ev

        self._side.wait_stream(main)
        if self.cp > 1:
            fetch(1)
        for i in range(self.cp):
            if i == 0:
                kk, vv = k_sym, v_sym
            else:
                slot = i & 1
                main.wait_event(ready[slot])
                kk, vv = stage[slot]
            o, lse = ops.attention(q, kk, vv, mask=ops.MASK_FULL, return_lse=True)
            if i > 0:
                ev = torch.cuda.Event()
                ev.record(main)
                consumed[i & 1] = ev
            if i + 1 < self.cp and i >= 1:  # hop 1 was requested before the loop
                fetch(i + 1)
            o_run, lse_run = merge_partial(o_run, lse_run, o, lse)
        main.wait_stream(self._side)
        self.sg.barrier(slot=6)  # peers are done reading this layer's shards
        return o_run.to(q.dtype)

    def attend(self, q, k, v, mask: int, n_ar: int = 0):
        if mask != ops.MASK_FULL:
            raise NotImplementedError("ring-KV is implemented for the Generator's full attention")
        if self.fused and q.is_cuda and q.dtype == torch.bfloat16 and not torch.is_grad_enabled():
            return self._attend_fused(q, k, v, mask)
        return self._attend_gloo(q, k, v, mask)

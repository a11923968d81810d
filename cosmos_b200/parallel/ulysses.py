"""Ulysses context parallelism: activations are sharded along the sequence everywhere except
inside attention, where each rank holds all tokens of H/cp heads (reference: `--cp-size`,
evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb:624,645, and `--ulysses-degree`,
README.md:319).

Two implementations with the same interface:
  * `fused=False` (also the CPU/gloo path and the autograd path used in training): NCCL/gloo
    `all_to_all_single` before and after a local attention. This is the baseline.
  * `fused=True` (CUDA bf16, head_dim 128, inference): no separate collective at all. The QKV
    GEMM's epilogue applies q/k RMSNorm + mRoPE and stores every head chunk directly into the
    owning rank's symmetric buffer over NVLink (sequence->head all-to-all), and the attention
    kernel's epilogue stores each block of output rows into the rank that owns those rows
    (head->sequence all-to-all). Two device-side group barriers per layer order the traffic.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..config import MoTConfig
from ..models.mot import KV, AttnContext, qkv_project_local
from .mesh import Mesh
from .symm import SymmGroup, symm_group


class _SeqToHead(torch.autograd.Function):
    """[B, S_loc, H, D] (all heads, local tokens) -> [B, S, H/cp, D] (local heads, all tokens)."""

    @staticmethod
    def forward(ctx, x, group, cp):
        ctx.group, ctx.cp = group, cp
        return _seq_to_head(x, group, cp)

    @staticmethod
    def backward(ctx, g):
        return _head_to_seq(g.contiguous(), ctx.group, ctx.cp), None, None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, cp):
        ctx.group, ctx.cp = group, cp
        return _head_to_seq(x, group, cp)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_head(g.contiguous(), ctx.group, ctx.cp), None, None


def _seq_to_head(x, group, cp):
    b, s_loc, h, d = x.shape
    send = x.reshape(b, s_loc, cp, h // cp, d).permute(2, 0, 1, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[src] = tokens of rank src for my heads
    return recv.permute(1, 0, 2, 3, 4).reshape(b, cp * s_loc, h // cp, d)


def _head_to_seq(x, group, cp):
    b, s, h_loc, d = x.shape
    s_loc = s // cp
    send = x.reshape(b, cp, s_loc, h_loc, d).permute(1, 0, 2, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[src] = my tokens for the heads owned by rank src
    return recv.permute(1, 2, 0, 3, 4).reshape(b, s_loc, cp * h_loc, d)


class UlyssesAttn(AttnContext):
    def __init__(self, cfg: MoTConfig, group, ranks, device, fused: bool = True):
        self.cfg = cfg
        self.group = group
        self.cp = len(ranks)
        self.rank = ranks.index(dist.get_rank())
        if cfg.n_kv_heads % self.cp or cfg.n_heads % self.cp:
            raise ValueError(f"Ulysses needs cp ({self.cp}) to divide the head counts "
                             f"({cfg.n_heads} q / {cfg.n_kv_heads} kv); use ring-KV instead")
        self.fused = bool(fused) and torch.device(device).type == "cuda" and cfg.head_dim == 128
        self.sg: Optional[SymmGroup] = symm_group(group, ranks, device) if self.fused else None
        self._ws: Dict = {}
        self._cur = None

    # ------------------------------------------------------------------ baseline path
    def _baseline_project(self, h, w, cos, sin, q_norm, k_norm, cfg, prefix):
        q, k, v = qkv_project_local(h, w, cos, sin, q_norm, k_norm, cfg)
        q = _SeqToHead.apply(q.contiguous(), self.group, self.cp)
        k = _SeqToHead.apply(k.contiguous(), self.group, self.cp)
        v = _SeqToHead.apply(v.contiguous(), self.group, self.cp)
        if prefix is not None:
            hk = cfg.n_kv_heads // self.cp
            sl = slice(self.rank * hk, (self.rank + 1) * hk)
            k = torch.cat([prefix[0][:, :, sl], k], dim=1)
            v = torch.cat([prefix[1][:, :, sl], v], dim=1)
        return q, k, v

    # ------------------------------------------------------------------ fused path
    def _workspace(self, b, s_loc, n_pre, like):
        key = (b, s_loc, n_pre)
        if key in self._ws:
            return self._ws[key]
        cfg, cp, r, sg = self.cfg, self.cp, self.rank, self.sg
        hq, hk, hd = cfg.n_heads // cp, cfg.n_kv_heads // cp, cfg.head_dim
        s = s_loc * cp
        es = 2
        q_bytes = b * s * hq * hd * es
        kv_bytes = b * (n_pre + s) * hk * hd * es
        o_bytes = b * s_loc * cfg.n_heads * hd * es
        q_off, k_off, v_off = 0, q_bytes, q_bytes + kv_bytes
        o_off = q_bytes + 2 * kv_bytes
        buf = sg.alloc(f"ulysses_{b}_{s_loc}_{n_pre}", o_off + o_bytes)
        qb = buf.view(q_off, (b, s, hq, hd), like.dtype)
        kb = buf.view(k_off, (b, n_pre + s, hk, hd), like.dtype)
        vb = buf.view(v_off, (b, n_pre + s, hk, hd), like.dtype)
        ob = buf.view(o_off, (b, s_loc, cfg.n_heads, hd), like.dtype)
        routes = []
        for bi in range(b):
            ptrs, lds = [], []
            for j in range(cfg.n_heads):
                owner, lh = divmod(j, hq)
                ptrs.append(buf.peer_addr(owner, q_off + ((bi * s + r * s_loc) * hq + lh) * hd * es))
                lds.append(hq * hd)
            for base in (k_off, v_off):
                for j in range(cfg.n_kv_heads):
                    owner, lh = divmod(j, hk)
                    ptrs.append(buf.peer_addr(owner, base + ((bi * (n_pre + s) + n_pre + r * s_loc) * hk + lh) * hd * es))
                    lds.append(hk * hd)
            routes.append((torch.tensor(ptrs, dtype=torch.int64, device=like.device),
                           torch.tensor(lds, dtype=torch.int64, device=like.device)))
        dest = torch.tensor([buf.peer_addr(p, o_off + r * hq * hd * es) for p in range(cp)],
                            dtype=torch.int64, device=like.device)
        self._ws[key] = (qb, kb, vb, ob, routes, dest)
        return self._ws[key]

    def qkv_project(self, h, w, cos, sin, q_norm, k_norm, cfg: MoTConfig, prefix: Optional[KV] = None):
        use_fused = (self.fused and h.is_cuda and h.dtype == torch.bfloat16 and not torch.is_grad_enabled())
        if not use_fused:
            self._cur = None
            return self._baseline_project(h, w, cos, sin, q_norm, k_norm, cfg, prefix)
        b, s_loc, _ = h.shape
        n_pre = 0 if prefix is None else prefix[0].shape[1]
        qb, kb, vb, ob, routes, dest = self._workspace(b, s_loc, n_pre, h)
        if prefix is not None:
            hk = cfg.n_kv_heads // self.cp
            sl = slice(self.rank * hk, (self.rank + 1) * hk)
            kb[:, :n_pre].copy_(prefix[0][:, :, sl])
            vb[:, :n_pre].copy_(prefix[1][:, :, sl])
        gq = q_norm if cfg.qk_norm else None
        gk = k_norm if cfg.qk_norm else None
        for bi in range(b):
            ops.gemm_qkv_rope(h[bi], w, None, cos, sin, gq, gk, cfg.n_heads, cfg.n_kv_heads, cfg.rms_eps,
                              routes[bi][0], routes[bi][1])
        self.sg.barrier(slot=0)  # every rank's q/k/v stores have landed
        self._cur = (ob, dest, s_loc)
        return qb, kb, vb

    def attend(self, q, k, v, mask: int, n_ar: int = 0):
        if self._cur is None:
            o, _ = ops.attention(q, k, v, mask=mask, n_ar=n_ar)
            return _HeadToSeq.apply(o.contiguous(), self.group, self.cp)
        ob, dest, s_loc = self._cur
        hq = self.cfg.n_heads // self.cp
        ops.attention(q, k, v, mask=mask, n_ar=n_ar, dest_ptr=dest, rows_per_dest=s_loc, out=ob[:, :, :hq])
        self.sg.barrier(slot=1)  # every rank's output rows have landed; q/k/v buffers are free again
        self._cur = None
        return ob


def make_cp_context(cfg: MoTConfig, mesh: Mesh, fused: bool = True) -> AttnContext:
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    ranks = mesh.group_ranks["cp"]
    if mesh.pc.cp_mode == "ring":
        from .ring import RingAttn
        return RingAttn(cfg, mesh.group("cp"), ranks, device, fused)
    return UlyssesAttn(cfg, mesh.group("cp"), ranks, device, fused)

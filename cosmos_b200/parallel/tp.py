"""Tensor parallelism with sequence parallelism (Megatron layout): QKV and FC1 are split by
output columns (heads / FFN units), out-proj and FC2 by input columns; between the TP regions
activations are sharded along the sequence, so each all-reduce becomes an all-gather before the
column-parallel GEMM and a reduce-scatter after the row-parallel GEMM (reference:
`--tensor-parallel-size`, README.md:312-321; the published 4x/8x numbers use TP,
inference_benchmarks.md:130).

Paths:
  * baseline (any device): `all_gather_into_tensor` / `reduce_scatter_tensor` / `all_reduce`.
  * fused (CUDA bf16):
      AG -> GEMM : the peers' sequence shards are pulled block by block into local memory by a copy
                   kernel on a side stream (plain peer loads, every byte crosses NVLink once) while
                   the tcgen05 GEMM already runs on the blocks that have arrived (own block first).
      GEMM -> RS : the GEMM runs once per destination row block and its epilogue stores the partial
                   tile straight into the owning rank's partial buffer (peer stores); after one
                   device barrier the owner sums the tp partials and applies the gated residual.
      decode     : activations are tiny, so the row-parallel outputs are summed by the one-shot
                   all-reduce kernel (every rank reads all peers' buffers after a barrier).
Attention itself needs no communication: each rank owns H/tp heads for the whole sequence, which
is also the Ulysses layout, so "TP + Ulysses over heads" shares this code path.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..config import MoTConfig
from ..models.mot import KV, AttnContext
from .symm import symm_group


def tp_local_config(cfg: MoTConfig, tp: int) -> MoTConfig:
    """The configuration of ONE tensor-parallel rank's model shard: 1/tp of the heads and of the FFN units, everything
    else (width, layers, vocabulary, embeddings, modulation tables) as in `cfg`. A `MoTModel` built from it holds
    only that rank's slice of every block weight (Cosmos3-Super on 8 ranks: 16 GB of block weights per GPU instead
    of 128 GB), and `TPContext(cfg, ..., presliced=True)` runs it."""
    import dataclasses
    if cfg.n_heads % tp or cfg.n_kv_heads % tp or cfg.ffn_dim % tp:
        raise ValueError("tp must divide the head counts and the FFN width")
    return dataclasses.replace(cfg, n_heads=cfg.n_heads // tp, n_kv_heads=cfg.n_kv_heads // tp,
                               ffn_dim=cfg.ffn_dim // tp)


def tp_slice_rows(name: str, cfg: MoTConfig, tp: int, rank: int):
    """Which part of a full block weight `name` belongs to `rank`: ("rows", [(start, stop), ...]) for weights split by
    output rows (wqkv: the rank's q, k and v head blocks; w_gate_up: its gate and up blocks), ("cols", (start, stop))
    for weights split by input columns (wo, w_down), None for replicated tensors. Used to read a rank's shard straight
    from a checkpoint (`ckpt/safetensors_io.py::read_range` for row blocks)."""
    hd = cfg.head_dim
    if name == "wqkv":
        hq, hk = cfg.n_heads // tp, cfg.n_kv_heads // tp
        q0, k0, v0 = 0, cfg.q_dim, cfg.q_dim + cfg.kv_dim
        return "rows", [(q0 + rank * hq * hd, q0 + (rank + 1) * hq * hd), (k0 + rank * hk * hd, k0 + (rank + 1) * hk * hd),
                        (v0 + rank * hk * hd, v0 + (rank + 1) * hk * hd)]
    if name == "w_gate_up":
        f = cfg.ffn_dim // tp
        return "rows", [(rank * f, (rank + 1) * f), (cfg.ffn_dim + rank * f, cfg.ffn_dim + (rank + 1) * f)]
    if name == "wo":
        c = cfg.q_dim // tp
        return "cols", (rank * c, (rank + 1) * c)
    if name == "w_down":
        f = cfg.ffn_dim // tp
        return "cols", (rank * f, (rank + 1) * f)
    return None


def shard_full_model(full, local, cfg: MoTConfig, tp: int, rank: int) -> None:
    """Copies `rank`'s slices of a full `MoTModel` into a model built from `tp_local_config` (tests, and loading a
    checkpoint that was read in full); replicated tensors are copied whole."""
    with torch.no_grad():
        for tname in ("ar", "dm"):
            ft, lt = getattr(full, tname, None), getattr(local, tname, None)
            if ft is None or lt is None:
                continue
            for fl, ll in zip(ft.layers, lt.layers):
                fv, lv = fl.views(), ll.views()
                for name, dst in lv.items():
                    how = tp_slice_rows(name, cfg, tp, rank)
                    if how is None:
                        dst.copy_(fv[name])
                    elif how[0] == "rows":
                        dst.copy_(torch.cat([fv[name][a:b] for a, b in how[1]]))
                    else:
                        dst.copy_(fv[name][:, how[1][0]:how[1][1]])
        skip = {n for n, _ in local.named_parameters() if ".layers." in n}
        fp = dict(full.named_parameters())
        for n, p in local.named_parameters():
            if n not in skip and n in fp and fp[n].shape == p.shape:
                p.copy_(fp[n])


class TPContext(AttnContext):
    def __init__(self, cfg: MoTConfig, group, ranks: List[int], device, fused: bool = True,
                 sequence_parallel: bool = True, presliced: bool = False):
        """`cfg` is always the FULL model's configuration. `presliced`: the model that runs under this context was
        built from `tp_local_config(cfg, tp)`, so its weights (and the K/V it caches) are this rank's slices already."""
        self.cfg, self.group = cfg, group
        self.presliced = bool(presliced)
        self._ranks = list(ranks)
        self.tp = len(ranks)
        self.rank = ranks.index(dist.get_rank()) if dist.is_initialized() else 0
        if cfg.n_kv_heads % self.tp or cfg.n_heads % self.tp or cfg.ffn_dim % self.tp:
            raise ValueError("tp must divide the head counts and the FFN width")
        self.device = torch.device(device)
        self.sp = sequence_parallel
        self.fused = bool(fused) and self.device.type == "cuda" and self.tp > 1
        self.sg = symm_group(group, ranks, device) if self.fused else None
        self._side = torch.cuda.Stream() if self.fused else None
        self._wcache: Dict = {}
        self._ws: Dict = {}
        self._ar_epoch = 0
        self._arn_parity = 0

    @property
    def cp(self) -> int:
        """Sequence-parallel degree seen by the engine (tokens are sharded like context parallelism)."""
        return self.tp if self.sp else 1

    # ------------------------------------------------------------------ weight slices
    def _slice(self, w: torch.Tensor, kind: str) -> torch.Tensor:
        """Local part of a full weight. Cached per storage so inference slices once."""
        if self.presliced:
            return w
        key = (w.data_ptr(), kind, tuple(w.shape))
        if key in self._wcache and not torch.is_grad_enabled():
            return self._wcache[key]
        cfg, tp, r = self.cfg, self.tp, self.rank
        hd = cfg.head_dim
        if kind == "qkv":
            hq, hk = cfg.n_heads // tp, cfg.n_kv_heads // tp
            q0, k0, v0 = 0, cfg.q_dim, cfg.q_dim + cfg.kv_dim
            out = torch.cat([w[q0 + r * hq * hd:q0 + (r + 1) * hq * hd],
                             w[k0 + r * hk * hd:k0 + (r + 1) * hk * hd],
                             w[v0 + r * hk * hd:v0 + (r + 1) * hk * hd]])
        elif kind == "wo":
            c = cfg.q_dim // tp
            out = w[:, r * c:(r + 1) * c].contiguous()
        elif kind == "gate_up":
            f = cfg.ffn_dim // tp
            out = torch.cat([w[r * f:(r + 1) * f], w[cfg.ffn_dim + r * f:cfg.ffn_dim + (r + 1) * f]])
        elif kind == "down":
            f = cfg.ffn_dim // tp
            out = w[:, r * f:(r + 1) * f].contiguous()
        else:
            raise KeyError(kind)
        if not torch.is_grad_enabled():
            self._wcache[key] = out
        return out

    # ------------------------------------------------------------------ collectives
    def _all_gather_seq(self, x: torch.Tensor) -> torch.Tensor:
        """[B, S/tp, d] -> [B, S, d]"""
        if self.tp == 1 or not self.sp:
            return x
        b, s_loc, d = x.shape
        if self.fused and x.is_cuda and x.dtype == torch.bfloat16 and b == 1 and not torch.is_grad_enabled():
            return self._ag_fused_start(x)
        parts = torch.empty(self.tp * b, s_loc, d, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(parts, x.contiguous(), group=self.group)
        return parts.view(self.tp, b, s_loc, d).permute(1, 0, 2, 3).reshape(b, self.tp * s_loc, d)

    def _ag_fused_start(self, x: torch.Tensor) -> torch.Tensor:
        """Publishes the local shard and launches the block-wise pulls on the side stream. Returns
        the full buffer; `self._ag_events[r]` is recorded when block r is complete, and the GEMM
        wrapper consumes the blocks in arrival order."""
        b, s_loc, d = x.shape
        key = ("ag", s_loc, d)
        if key not in self._ws:
            nb = s_loc * d * 2
            buf = self.sg.alloc(f"tp_ag_{s_loc}_{d}", nb)
            sym = buf.view(0, (s_loc, d), x.dtype)
            ptrs = [torch.tensor([buf.peer_addr(r)], dtype=torch.int64, device=x.device) for r in range(self.tp)]
            full = torch.empty(self.tp * s_loc, d, dtype=x.dtype, device=x.device)
            self._ws[key] = (sym, ptrs, full, nb)
        sym, ptrs, full, nb = self._ws[key]
        sym.copy_(x[0])
        self.sg.barrier(slot=7)
        main = torch.cuda.current_stream()
        full[self.rank * s_loc:(self.rank + 1) * s_loc].copy_(x[0])
        self._side.wait_stream(main)
        self._ag_events = {}
        order = [(self.rank + i) % self.tp for i in range(1, self.tp)]
        with torch.cuda.stream(self._side):
            for r in order:
                torch.ops.cosmos_b200.allgather_pull(ptrs[r], 1, full[r * s_loc:(r + 1) * s_loc], nb)
                ev = torch.cuda.Event()
                ev.record(self._side)
                self._ag_events[r] = ev
        self._ag_order = [self.rank] + order
        self._ag_s_loc = s_loc
        return full[None]

    def _gemm_rowblocks(self, x_full: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
        """Column-parallel GEMM on a gathered input; with a fused gather in flight, runs block by
        block as the peers' rows arrive."""
        ev = getattr(self, "_ag_events", None)
        if not ev:
            return ops.gemm(x_full, w, **kw)
        s_loc = self._ag_s_loc
        n_out = w.shape[0] // 2 if kw.get("epi") == ops.EPI_SWIGLU else w.shape[0]
        out = torch.empty(x_full.shape[0], x_full.shape[1], n_out, dtype=x_full.dtype, device=x_full.device)
        main = torch.cuda.current_stream()
        for r in self._ag_order:
            if r in ev:
                main.wait_event(ev[r])
            ops.gemm(x_full[0, r * s_loc:(r + 1) * s_loc], w, out=out[0, r * s_loc:(r + 1) * s_loc], **kw)
        return out

    def _ag_done(self):
        if getattr(self, "_ag_events", None):
            torch.cuda.current_stream().wait_stream(self._side)
            self._ag_events = None

    def _reduce_scatter_seq(self, partial_fn, s: int, d: int, resid, gate, rows_per_batch, like) -> torch.Tensor:
        """Row-parallel GEMM + reduce-scatter along the sequence + gated residual.
        `partial_fn(row_slice, out)` computes the partial product of a block of rows (into `out`
        when given)."""
        tp, r = self.tp, self.rank
        if tp == 1:
            return ops.gated_residual(resid, partial_fn(slice(0, s), None), gate, rows_per_batch)
        s_loc = s // tp
        if self.fused and like.is_cuda and like.dtype == torch.bfloat16 and not torch.is_grad_enabled():
            b = like.shape[0]
            key = ("rs", b, s_loc, d)
            if key not in self._ws:
                nb = b * s_loc * d * 2
                buf = self.sg.alloc(f"tp_rs_{b}_{s_loc}_{d}", tp * nb)
                mine = buf.view(0, (tp, b, s_loc, d), like.dtype)
                peers = [buf._handle.get_buffer(p, (b, s_loc, d), like.dtype, r * b * s_loc * d) for p in range(tp)]
                self._ws[key] = (mine, peers)
            mine, peers = self._ws[key]
            for i in range(tp):
                p = (r + i) % tp  # own block first, then staggered so that no peer is hit by all ranks at once
                partial_fn(slice(p * s_loc, (p + 1) * s_loc), peers[p])
            self.sg.barrier(slot=8)
            # one kernel: sum of the tp partial products (fp32) + gate + residual
            out = torch.ops.cosmos_b200.sum_partials_gated_residual(
                mine, resid, gate, rows_per_batch if gate is not None else 0).view(resid.shape)
            self.sg.barrier(slot=9)  # partial buffers may be overwritten again
            return out
        part = partial_fn(slice(0, s), None)
        b = part.shape[0]
        shard = torch.empty(b, s_loc, d, dtype=part.dtype, device=part.device)
        inp = part.reshape(b, tp, s_loc, d).permute(1, 0, 2, 3).reshape(tp * b, s_loc, d).contiguous()
        dist.reduce_scatter_tensor(shard, inp, group=self.group)
        return ops.gated_residual(resid, shard, gate, rows_per_batch)

    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp == 1:
            return x
        if self.fused and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0 and x.numel() <= (1 << 21):
            key = ("ar", x.numel())
            if key not in self._ws:
                buf = self.sg.alloc(f"tp_ar_{x.numel()}", x.numel() * 2)
                self._ws[key] = (buf.view(0, (x.numel(),), x.dtype),
                                 torch.tensor(buf.peer_ptrs, dtype=torch.int64, device=x.device))
            mine, ptrs = self._ws[key]
            mine.copy_(x.reshape(-1))
            out = torch.empty_like(x)
            # epochs of signal slots 16..47 (one row per block) are tracked on the device (the group's counters,
            # shared by every user of these slots), so the call is CUDA-graph safe
            torch.ops.cosmos_b200.allreduce_oneshot(ptrs, self.sg.pads_dev, out.view(-1), self.rank, self.tp, 16, 0,
                                                    self.sg.counters)
            return out
        y = x.contiguous()
        dist.all_reduce(y, group=self.group)
        return y

    def gemm_allreduce_norm(self, a: torch.Tensor, w: torch.Tensor, resid: Optional[torch.Tensor],
                            gamma: Optional[torch.Tensor], eps: float, want_norm: bool = True):
        """Row-parallel projection of a decode step in two launches: x_new = resid + sum over ranks of (a w^T) and
        h = rmsnorm(x_new) * gamma -> (h, x_new). Fused path: the GEMM leaves its split-K partial sums, and ONE
        kernel reduces them into this rank's symmetric buffer, meets the peers on the device, sums the ranks'
        buffers (multimem.ld_reduce through the NVLink switch when the buffer has a multicast mapping, else peer
        loads), adds the residual and applies the norm. Two buffers alternate between consecutive calls, which is
        what lets the kernel do without a trailing barrier; `begin_step` must open every step / CUDA graph."""
        m = a.numel() // a.shape[-1]
        n = w.shape[0]
        if (self.tp > 1 and self.fused and a.is_cuda and a.dtype == torch.bfloat16 and n % 8 == 0 and n <= 8192
                and not torch.is_grad_enabled()):
            key = ("arn", m, n)
            if key not in self._ws:
                entries = []
                for i in range(2):
                    buf = self.sg.alloc(f"tp_arn_{m}_{n}_{i}", m * n * 2)
                    entries.append((buf.view(0, (m, n), a.dtype),
                                    torch.tensor(buf.peer_ptrs, dtype=torch.int64, device=a.device),
                                    self.sg.use_multicast(buf)))
                self._ws[key] = entries
            self._arn_parity ^= 1
            own, ptrs, mc = self._ws[key][self._arn_parity]
            h, x_new = torch.ops.cosmos_b200.gemm_allreduce_norm(
                a, w, resid, gamma, eps, ptrs, mc, own, self.sg.pads_dev, self.rank, self.tp, 16, self.sg.counters,
                want_norm)
            shape = tuple(a.shape[:-1]) + (n,)
            return h.view(shape), x_new.view(shape)
        y = self._all_reduce(ops.gemm(a, w))
        if resid is None:
            return (ops.rmsnorm(y, gamma, eps)[0] if want_norm else y), y
        if not want_norm:
            x_new = resid + y
            return x_new, x_new
        return ops.rmsnorm(y, gamma, eps, residual=resid)

    def begin_step(self) -> None:
        """Opens a decode step (or its CUDA graph): one device barrier, after which every peer has finished
        reading the buffers of the previous step, and the buffer alternation restarts."""
        self._arn_parity = 0
        if self.tp > 1 and self.fused:
            self.sg.barrier_counted(slot=15)

    # ------------------------------------------------------------------ AttnContext interface
    def prefill_context(self) -> "TPContext":
        """The same ranks and buffers without sequence parallelism (every rank holds the whole, short sequence and the
        row-parallel outputs are all-reduced): how the prompt runs through a pre-sliced AR tower."""
        if not self.sp:
            return self
        if getattr(self, "_prefill", None) is None:
            c = TPContext(self.cfg, self.group, self._ranks, self.device, fused=self.fused, sequence_parallel=False,
                          presliced=self.presliced)
            self._prefill = c
        return self._prefill

    def qkv_project(self, h, w, cos, sin, q_norm, k_norm, cfg: MoTConfig, prefix: Optional[KV] = None):
        cfg = self.cfg   # head counts come from the full configuration (the caller's may be the rank-local one)
        wl = self._slice(w, "qkv")
        x = self._all_gather_seq(h)
        b, s, _ = x.shape
        hq, hk, hd = cfg.n_heads // self.tp, cfg.n_kv_heads // self.tp, cfg.head_dim
        gq = q_norm if cfg.qk_norm else None
        gk = k_norm if cfg.qk_norm else None
        # cos/sin are given for the local sequence shard; attention needs the full sequence
        cos_f, sin_f = self._full_rope(cos, sin)
        if x.is_cuda and x.dtype == torch.bfloat16 and hd == 128 and b == 1 and not torch.is_grad_enabled() \
                and ops.get_backend() == "own":
            # q/k RMS-norm and the rotary rotation run in the GEMM's epilogue, row block by row block as the
            # peers' sequence shards arrive
            qkv = self._gemm_rowblocks_qkv(x, wl, cos_f, sin_f, gq, gk, hq, hk).view(b, s, hq + 2 * hk, hd)
            self._ag_done()
            q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
        else:
            qkv = self._gemm_rowblocks(x, wl).view(b, s, hq + 2 * hk, hd)
            self._ag_done()
            q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
            if q.is_cuda and q.dtype == torch.bfloat16 and hd == 128:
                q = ops.mrope(q.contiguous(), cos_f, sin_f, gq, cfg.rms_eps)
                k = ops.mrope(k.contiguous(), cos_f, sin_f, gk, cfg.rms_eps)
            else:
                q = ops.ref.mrope(q, cos_f, sin_f, gq, cfg.rms_eps)
                k = ops.ref.mrope(k, cos_f, sin_f, gk, cfg.rms_eps)
        if prefix is not None:
            sl = slice(None) if (self.presliced or prefix[0].shape[2] == hk) else slice(self.rank * hk, (self.rank + 1) * hk)
            k = torch.cat([prefix[0][:, :, sl], k], dim=1)
            v = torch.cat([prefix[1][:, :, sl], v], dim=1)
        return q, k, v

    def _gemm_rowblocks_qkv(self, x_full, w, cos, sin, gq, gk, hq, hk) -> torch.Tensor:
        """QKV projection with the fused norm + rotary epilogue on a gathered input [1, S, d] -> [1, S, (hq + 2 hk) * 128];
        with a fused gather in flight it runs block by block in arrival order, each block with its rows of the
        rotary tables."""
        eps = self.cfg.rms_eps
        ev = getattr(self, "_ag_events", None)
        if not ev:
            return ops.gemm_qkv_rope(x_full[0], w, None, cos, sin, gq, gk, hq, hk, eps)[None]
        s_loc = self._ag_s_loc
        out = torch.empty(1, x_full.shape[1], w.shape[0], dtype=x_full.dtype, device=x_full.device)
        main = torch.cuda.current_stream()
        for r in self._ag_order:
            if r in ev:
                main.wait_event(ev[r])
            rows = slice(r * s_loc, (r + 1) * s_loc)
            ops.gemm_qkv_rope(x_full[0, rows], w, None, cos[rows].contiguous(), sin[rows].contiguous(), gq, gk, hq, hk, eps,
                              out=out[0, rows])
        return out

    def _full_rope(self, cos, sin):
        if self.tp == 1 or not self.sp:
            return cos, sin
        key = ("rope", cos.data_ptr())
        if key not in self._ws:
            c = torch.empty(self.tp * cos.shape[0], cos.shape[1], dtype=cos.dtype, device=cos.device)
            s = torch.empty_like(c)
            dist.all_gather_into_tensor(c, cos.contiguous(), group=self.group)
            dist.all_gather_into_tensor(s, sin.contiguous(), group=self.group)
            self._ws[key] = (c, s)
        return self._ws[key]

    def out_project(self, o, w, resid, gate, rows_per_batch):
        wl = self._slice(w, "wo")
        if not self.sp:
            y = self._all_reduce(ops.gemm(o, wl))
            return ops.gated_residual(resid, y, gate, rows_per_batch)
        b, s, _ = o.shape

        def partial(rows, out):
            return ops.gemm(o[:, rows], wl, out=out)

        return self._reduce_scatter_seq(partial, s, w.shape[0], resid, gate, rows_per_batch, o)

    def mlp(self, h, w_gate_up, w_down, resid, gate, rows_per_batch):
        wg, wd = self._slice(w_gate_up, "gate_up"), self._slice(w_down, "down")
        if not self.sp:
            a = ops.gemm(h, wg, epi=ops.EPI_SWIGLU)
            y = self._all_reduce(ops.gemm(a, wd))
            return ops.gated_residual(resid, y, gate, rows_per_batch)
        x = self._all_gather_seq(h)
        a = self._gemm_rowblocks(x, wg, epi=ops.EPI_SWIGLU)
        self._ag_done()
        b, s, _ = a.shape

        def partial(rows, out):
            return ops.gemm(a[:, rows], wd, out=out)

        return self._reduce_scatter_seq(partial, s, w_down.shape[0], resid, gate, rows_per_batch, a)

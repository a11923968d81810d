"""Mixture-of-Transformers backbone: an autoregressive (AR / Reasoner) tower and a diffusion
(DM / Generator) tower with separate weights that meet in one attention per layer.

Attention semantics (reference README.md:74 and the architecture diagram
cookbooks/cosmos3/cosmos3-model-architecture.png):
  Reasoner  : Attn(Q_AR, K_AR, V_AR), causal.
  Generator : Attn(Q_DM, [K_AR; K_DM], [V_AR; V_DM]), full. AR rows never see DM keys, so the
              AR tower's K/V of the prompt are computed once and reused by every denoise step.
  Joint     : one sequence [AR; DM] with the block mask (AR rows causal over AR keys, DM rows
              see everything) for training both towers together.

Each layer's parameters live in ONE flat tensor (views are cut out of it on use), which is the
unit that FSDP shards, all-gathers and reduce-scatters.

Hot ops go through `cosmos_b200.ops` (sm_100a kernels on CUDA, plain PyTorch on CPU):
QKV GEMM with q/k-RMSNorm + mRoPE epilogue, flash attention, out-proj / FC2 GEMM with gated
residual epilogue, FC1 GEMM with SwiGLU epilogue, AdaLN-modulated RMSNorm.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import MoTConfig
from . import rope

KV = Tuple[torch.Tensor, torch.Tensor]


def layer_spec(cfg: MoTConfig, is_dm: bool) -> "OrderedDict[str, Tuple[int, ...]]":
    d = cfg.d_model
    spec = OrderedDict()
    spec["norm1"] = (d,)
    spec["wqkv"] = (cfg.qkv_dim, d)
    spec["q_norm"] = (cfg.head_dim,)
    spec["k_norm"] = (cfg.head_dim,)
    spec["wo"] = (d, cfg.q_dim)
    spec["norm2"] = (d,)
    spec["w_gate_up"] = (2 * cfg.ffn_dim, d)
    spec["w_down"] = (d, cfg.ffn_dim)
    if is_dm:
        spec["mod_table"] = (6, d)
    return spec


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class _FlatSplit(torch.autograd.Function):
    """flat [n] -> the named views of a `FlatLayer`; backward gathers the views' gradients into one flat tensor."""

    @staticmethod
    def forward(ctx, flat: torch.Tensor, layer: "FlatLayer"):
        ctx.layer = layer
        ctx.meta = (flat.shape, flat.dtype, flat.device)
        return tuple(flat[off:off + n].view(layer.spec[name]) for name, (off, n) in layer.offsets.items())

    @staticmethod
    def backward(ctx, *grads):
        shape, dtype, device = ctx.meta
        g = torch.zeros(shape, dtype=dtype, device=device)
        for (name, (off, n)), gv in zip(ctx.layer.offsets.items(), grads):
            if gv is not None:
                g[off:off + n].copy_(gv.reshape(-1))
        return g, None


class FlatLayer(nn.Module):
    """One transformer layer's parameters as a single flat tensor with named views.

    Every view starts on a 128-element boundary so that TMA descriptors built on a view are
    16-byte aligned for any dtype; `pad_to` lets FSDP make the flat length divisible by its
    shard count.
    """

    def __init__(self, spec: "OrderedDict[str, Tuple[int, ...]]", dtype, device, pad_to: int = 128):
        super().__init__()
        self.spec = spec
        self.offsets: Dict[str, Tuple[int, int]] = {}
        off = 0
        for name, shape in spec.items():
            n = math.prod(shape)
            self.offsets[name] = (off, n)
            off = _round_up(off + n, 128)
        self.numel_padded = _round_up(off, pad_to)
        self.flat = nn.Parameter(torch.zeros(self.numel_padded, dtype=dtype, device=device))

    def views(self, flat: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        flat = self.flat if flat is None else flat
        if torch.is_grad_enabled() and flat.requires_grad:
            # one autograd node for all views: its backward writes every view's gradient into ONE flat gradient
            # (plain slicing would build a full-size zero tensor per view and add them up pairwise)
            outs = _FlatSplit.apply(flat, self)
            return dict(zip(self.offsets.keys(), outs))
        return {name: flat[off:off + n].view(self.spec[name]) for name, (off, n) in self.offsets.items()}

    @torch.no_grad()
    def init_weights(self, std: float, generator: Optional[torch.Generator] = None) -> None:
        v = self.views()
        for name, t in v.items():
            if name in ("norm1", "norm2", "q_norm", "k_norm"):
                t.fill_(1.0)
            elif name == "mod_table":
                t.zero_()
            else:
                t.normal_(0.0, std, generator=generator)


class Tower(nn.Module):
    def __init__(self, cfg: MoTConfig, is_dm: bool, dtype, device, pad_to: int = 128):
        super().__init__()
        self.cfg, self.is_dm = cfg, is_dm
        spec = layer_spec(cfg, is_dm)
        self.layers = nn.ModuleList([FlatLayer(spec, dtype, device, pad_to) for _ in range(cfg.n_layers)])


def sinusoidal_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    """t [B] in [0, 1] (scaled by 1000 as in diffusion timestep embeddings) -> [B, dim] fp32."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    args = t.float()[:, None] * 1000.0 * freqs[None]
    return torch.cat([args.cos(), args.sin()], dim=-1)


# --------------------------------------------------------------------------- attention plumbing
class AttnContext:
    """How a layer runs its attention. The default is local attention; the context-parallel
    wrappers in `cosmos_b200.parallel` subclass this to insert the Ulysses all-to-all or the
    ring-KV schedule, and `WorkspaceAttn` below removes the K/V concatenation copies.
    `prefix` is a (K, V) pair that is prepended to this call's keys/values (the cached AR
    tokens for a Generator layer, the KV cache for a Reasoner layer)."""

    def qkv_project(self, h, w, cos, sin, q_norm, k_norm, cfg: MoTConfig, prefix: Optional[KV] = None):
        q, k, v = qkv_project_local(h, w, cos, sin, q_norm, k_norm, cfg)
        if prefix is not None:
            k = torch.cat([prefix[0], k], dim=1)
            v = torch.cat([prefix[1], v], dim=1)
        return q, k, v

    def attend(self, q, k, v, mask: int, n_ar: int = 0):
        o, _ = ops.attention(q, k, v, mask=mask, n_ar=n_ar)
        return o

    def out_project(self, o, w, resid, gate, rows_per_batch):
        return ops.gemm(o, w, None, ops.EPI_GATED_RESID, resid, gate, rows_per_batch)

    def mlp(self, h, w_gate_up, w_down, resid, gate, rows_per_batch):
        a = ops.gemm(h, w_gate_up, epi=ops.EPI_SWIGLU)
        return ops.gemm(a, w_down, None, ops.EPI_GATED_RESID, resid, gate, rows_per_batch)


class WorkspaceAttn(AttnContext):
    """Inference-time context for CUDA bf16 / head_dim 128: the QKV GEMM's epilogue writes q, k, v
    straight into preallocated buffers through its routing table, with k and v landing behind
    the prefix rows of a [B, n_prefix + S, Hkv, 128] buffer, so no concatenation copy is made.
    Buffers are reused by every layer and every step (not usable under autograd)."""

    def __init__(self):
        self._ws: Dict = {}

    def _buffers(self, b, s, n_pre, cfg, like):
        key = (b, s, n_pre, like.device)
        if key not in self._ws:
            hq, hk, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
            qb = torch.empty(b, s, hq, hd, dtype=like.dtype, device=like.device)
            kb = torch.empty(b, n_pre + s, hk, hd, dtype=like.dtype, device=like.device)
            vb = torch.empty_like(kb)
            routes = []
            for bi in range(b):
                ptrs = ([qb[bi].data_ptr() + j * hd * 2 for j in range(hq)]
                        + [kb[bi, n_pre:].data_ptr() + j * hd * 2 for j in range(hk)]
                        + [vb[bi, n_pre:].data_ptr() + j * hd * 2 for j in range(hk)])
                lds = [hq * hd] * hq + [hk * hd] * (2 * hk)
                routes.append((torch.tensor(ptrs, dtype=torch.int64, device=like.device),
                               torch.tensor(lds, dtype=torch.int64, device=like.device)))
            self._ws[key] = (qb, kb, vb, routes)
        return self._ws[key]

    def qkv_project(self, h, w, cos, sin, q_norm, k_norm, cfg: MoTConfig, prefix: Optional[KV] = None):
        if (not (h.is_cuda and h.dtype == torch.bfloat16 and cfg.head_dim == 128) or torch.is_grad_enabled()
                or ops.get_backend() == "library"):
            return super().qkv_project(h, w, cos, sin, q_norm, k_norm, cfg, prefix)
        b, s, _ = h.shape
        n_pre = 0 if prefix is None else prefix[0].shape[1]
        qb, kb, vb, routes = self._buffers(b, s, n_pre, cfg, h)
        if prefix is not None:
            kb[:, :n_pre].copy_(prefix[0])
            vb[:, :n_pre].copy_(prefix[1])
        gq = q_norm if cfg.qk_norm else None
        gk = k_norm if cfg.qk_norm else None
        for bi in range(b):
            ops.gemm_qkv_rope(h[bi], w, None, cos, sin, gq, gk, cfg.n_heads, cfg.n_kv_heads, cfg.rms_eps,
                              routes[bi][0], routes[bi][1])
        return qb, kb, vb


def qkv_project_local(h, w, cos, sin, q_norm, k_norm, cfg: MoTConfig):
    """[B, S, d] -> q [B, S, Hq, hd], k, v [B, S, Hkv, hd] with q/k RMSNorm and mRoPE applied."""
    b, s, _ = h.shape
    hq, hk, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    gq = q_norm if cfg.qk_norm else None
    gk = k_norm if cfg.qk_norm else None
    if hd == 128 and h.is_cuda and h.dtype == torch.bfloat16 and not ops._grad_needed(h, w, q_norm, k_norm):
        qkv = ops.gemm_qkv_rope(h.reshape(b * s, -1), w, None, cos, sin, gq, gk, hq, hk, cfg.rms_eps)
        qkv = qkv.view(b, s, hq + 2 * hk, hd)
        return qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
    qkv = ops.gemm(h, w).view(b, s, hq + 2 * hk, hd)
    if hd == 128 and ops._train_cuda(qkv, q_norm, k_norm):
        # training on CUDA: norm + rotary + q/k/v split as one autograd function on the kernels
        from ..ops import autograd as own
        q, k, v = own.qkv_post(qkv.reshape(b * s, hq + 2 * hk, hd), hq, cos, sin, gq, gk, cfg.rms_eps)
        return q.view(b, s, hq, hd), k.view(b, s, hk, hd), v.view(b, s, hk, hd)
    q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
    q = ops.ref.mrope(q, cos, sin, gq, cfg.rms_eps)
    k = ops.ref.mrope(k, cos, sin, gk, cfg.rms_eps)
    return q, k, v


LOCAL_ATTN = AttnContext()


def dm_modulation(t_mod: torch.Tensor, mod_table: torch.Tensor) -> List[torch.Tensor]:
    """t_mod [B, 6d] (shared projection of the timestep embedding) + per-layer table [6, d]
    -> six [B, d] tensors: shift1, scale1, gate1, shift2, scale2, gate2."""
    b = t_mod.shape[0]
    d = mod_table.shape[-1]
    m = (t_mod.view(b, 6, d).float() + mod_table.float()[None]).to(t_mod.dtype)
    return [m[:, i].contiguous() for i in range(6)]


def dm_block(cfg: MoTConfig, p: Dict[str, torch.Tensor], x, t_mod, cos, sin, ar_kv: Optional[KV],
             ctx: AttnContext = LOCAL_ATTN):
    """One Generator layer on DM tokens x [B, S, d]; ar_kv = this layer's cached AR (K, V)."""
    b, s, d = x.shape
    sh1, sc1, g1, sh2, sc2, g2 = dm_modulation(t_mod, p["mod_table"])
    h = ops.adaln_rmsnorm(x, p["norm1"], sh1, sc1, s, cfg.rms_eps)
    q, k, v = ctx.qkv_project(h, p["wqkv"], cos, sin, p["q_norm"], p["k_norm"], cfg, prefix=ar_kv)
    o = ctx.attend(q, k, v, ops.MASK_FULL)
    x = ctx.out_project(o.reshape(o.shape[0], o.shape[1], -1), p["wo"], x, g1, s)
    h = ops.adaln_rmsnorm(x, p["norm2"], sh2, sc2, s, cfg.rms_eps)
    return ctx.mlp(h, p["w_gate_up"], p["w_down"], x, g2, s)


def ar_block(cfg: MoTConfig, p: Dict[str, torch.Tensor], x, cos, sin, past: Optional[KV] = None,
             ctx: AttnContext = LOCAL_ATTN) -> Tuple[torch.Tensor, KV]:
    """One Reasoner layer on AR tokens x [B, S, d]; returns (x, (K, V) including `past`)."""
    b, s, d = x.shape
    h, _ = ops.rmsnorm(x, p["norm1"], cfg.rms_eps)
    q, k, v = ctx.qkv_project(h, p["wqkv"], cos, sin, p["q_norm"], p["k_norm"], cfg, prefix=past)
    o = ctx.attend(q, k, v, ops.MASK_CAUSAL)
    x = ctx.out_project(o.reshape(o.shape[0], o.shape[1], -1), p["wo"], x, None, s)
    h, _ = ops.rmsnorm(x, p["norm2"], cfg.rms_eps)
    x = ctx.mlp(h, p["w_gate_up"], p["w_down"], x, None, s)
    return x, (k, v)


def joint_block(cfg: MoTConfig, p_ar, p_dm, x_ar, x_dm, t_mod, cos_ar, sin_ar, cos_dm, sin_dm,
                ctx: AttnContext = LOCAL_ATTN):
    """One layer on the joint sequence [AR; DM]: per-modality weights, one attention with the
    MoT block mask."""
    b, s_ar, d = x_ar.shape
    s_dm = x_dm.shape[1]
    sh1, sc1, g1, sh2, sc2, g2 = dm_modulation(t_mod, p_dm["mod_table"])
    h_ar, _ = ops.rmsnorm(x_ar, p_ar["norm1"], cfg.rms_eps)
    h_dm = ops.adaln_rmsnorm(x_dm, p_dm["norm1"], sh1, sc1, s_dm, cfg.rms_eps)
    qa, ka, va = ctx.qkv_project(h_ar, p_ar["wqkv"], cos_ar, sin_ar, p_ar["q_norm"], p_ar["k_norm"], cfg)
    qd, kd, vd = ctx.qkv_project(h_dm, p_dm["wqkv"], cos_dm, sin_dm, p_dm["q_norm"], p_dm["k_norm"], cfg)
    q = torch.cat([qa, qd], dim=1)
    k = torch.cat([ka, kd], dim=1)
    v = torch.cat([va, vd], dim=1)
    o = ctx.attend(q, k, v, ops.MASK_MOT, n_ar=s_ar)
    oa, od = o[:, :s_ar].reshape(b, s_ar, -1), o[:, s_ar:].reshape(b, s_dm, -1)
    grouped = type(ctx) in (AttnContext, WorkspaceAttn)  # local execution: one grouped launch per projection
    if grouped:
        x_ar, x_dm = ops.gemm_grouped2(oa, p_ar["wo"], od, p_dm["wo"], ops.EPI_GATED_RESID, x_ar, x_dm, None, g1,
                                       s_ar, s_dm)
    else:
        x_ar = ctx.out_project(oa, p_ar["wo"], x_ar, None, s_ar)
        x_dm = ctx.out_project(od, p_dm["wo"], x_dm, g1, s_dm)
    h_ar, _ = ops.rmsnorm(x_ar, p_ar["norm2"], cfg.rms_eps)
    h_dm = ops.adaln_rmsnorm(x_dm, p_dm["norm2"], sh2, sc2, s_dm, cfg.rms_eps)
    if grouped:
        a_ar, a_dm = ops.gemm_grouped2(h_ar, p_ar["w_gate_up"], h_dm, p_dm["w_gate_up"], ops.EPI_SWIGLU)
        x_ar, x_dm = ops.gemm_grouped2(a_ar, p_ar["w_down"], a_dm, p_dm["w_down"], ops.EPI_GATED_RESID, x_ar, x_dm,
                                       None, g2, s_ar, s_dm)
    else:
        x_ar = ctx.mlp(h_ar, p_ar["w_gate_up"], p_ar["w_down"], x_ar, None, s_ar)
        x_dm = ctx.mlp(h_dm, p_dm["w_gate_up"], p_dm["w_down"], x_dm, g2, s_dm)
    return x_ar, x_dm


# --------------------------------------------------------------------------- the model
class MoTModel(nn.Module):
    def __init__(self, cfg: MoTConfig, dtype=torch.float32, device="cpu", towers: Sequence[str] = ("ar", "dm"),
                 pad_to: int = 128):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        kw = dict(dtype=dtype, device=device)
        self.has_ar, self.has_dm = "ar" in towers, "dm" in towers
        if self.has_ar:
            self.ar = Tower(cfg, False, dtype, device, pad_to)
            self.embed = nn.Parameter(torch.zeros(cfg.vocab_size, d, **kw))
            self.ar_norm = nn.Parameter(torch.ones(d, **kw))
            self.lm_head = nn.Parameter(torch.zeros(cfg.vocab_size, d, **kw))
        if self.has_dm:
            self.dm = Tower(cfg, True, dtype, device, pad_to)
            self.patch_in = nn.Parameter(torch.zeros(d, cfg.patch_dim, **kw))
            self.patch_in_b = nn.Parameter(torch.zeros(d, **kw))
            self.t_mlp1 = nn.Parameter(torch.zeros(d, cfg.t_embed_dim, **kw))
            self.t_mlp1_b = nn.Parameter(torch.zeros(d, **kw))
            self.t_mlp2 = nn.Parameter(torch.zeros(d, d, **kw))
            self.t_mlp2_b = nn.Parameter(torch.zeros(d, **kw))
            self.t_proj = nn.Parameter(torch.zeros(6 * d, d, **kw))
            self.final_mod = nn.Parameter(torch.zeros(2 * d, d, **kw))
            self.dm_norm = nn.Parameter(torch.ones(d, **kw))
            self.patch_out = nn.Parameter(torch.zeros(cfg.patch_dim, d, **kw))
            self.sound_in = nn.Parameter(torch.zeros(d, cfg.sound_latent_dim, **kw))
            self.sound_out = nn.Parameter(torch.zeros(cfg.sound_latent_dim, d, **kw))
            n_dom = len(cfg.action_domains)
            self.action_in = nn.Parameter(torch.zeros(n_dom, d, cfg.action_dim_max, **kw))
            self.action_out = nn.Parameter(torch.zeros(n_dom, cfg.action_dim_max, d, **kw))
            self.fps_embed = nn.Parameter(torch.zeros(64, d, **kw))
            self.cond_flag = nn.Parameter(torch.zeros(2, d, **kw))
        self.init_weights()

    @torch.no_grad()
    def init_weights(self, seed: Optional[int] = None, layer_seed: Optional[int] = None) -> None:
        """Random initialisation. `layer_seed` (tensor-parallel shards): the block weights are drawn from it, while the
        replicated tensors (embeddings, projections, heads) still come from `seed` and so agree on every rank."""
        std = self.cfg.init_std
        gen = None
        dev = next(self.parameters()).device
        if seed is not None:
            gen = torch.Generator(device=dev)
            gen.manual_seed(seed)
        lgen = gen
        if layer_seed is not None:
            lgen = torch.Generator(device=dev)
            lgen.manual_seed(layer_seed)
        for tower in ([self.ar] if self.has_ar else []) + ([self.dm] if self.has_dm else []):
            for layer in tower.layers:
                layer.init_weights(std, lgen)
        for name, p in self.named_parameters():
            if ".layers." in name:
                continue
            if name in ("ar_norm", "dm_norm"):
                p.fill_(1.0)
            elif name.endswith("_b"):
                p.zero_()
            else:
                p.normal_(0.0, std, generator=gen)

    # ---- AR / Reasoner -------------------------------------------------------------------
    def embed_tokens(self, ids: torch.Tensor) -> torch.Tensor:
        return F.embedding(ids, self.embed)

    def ar_forward(self, x: torch.Tensor, pos: torch.Tensor, past: Optional[List[KV]] = None,
                   ctx: AttnContext = LOCAL_ATTN, layer_params: Optional[Callable] = None,
                   deepstack: Optional[Sequence[torch.Tensor]] = None, vision_mask: Optional[torch.Tensor] = None
                   ) -> Tuple[torch.Tensor, List[KV]]:
        """x [B, S, d] embeddings, pos [3, S] -> (hidden [B, S, d] before the final norm, per-layer KV).
        `deepstack` (features [n_vision, d] from the vision encoder) are added to the output of layer i,
        i < len(deepstack), at the positions flagged by `vision_mask` [B, S]."""
        cfg = self.cfg
        cos, sin = rope.rope_tables(pos, cfg.head_dim, cfg.rope_theta, cfg.mrope_section)
        kvs: List[KV] = []
        for i, layer in enumerate(self.ar.layers):
            p = layer.views() if layer_params is None else layer_params("ar", i)
            x, kv = ar_block(cfg, p, x, cos, sin, None if past is None else past[i], ctx)
            kvs.append(kv)
            if deepstack is not None and vision_mask is not None and i < len(deepstack):
                n = int(vision_mask.sum())
                x = x.clone()
                x[vision_mask] = x[vision_mask] + deepstack[i].to(x.dtype).reshape(-1, x.shape[-1])[:n]
        return x, kvs

    def lm_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        h, _ = ops.rmsnorm(hidden, self.ar_norm, self.cfg.rms_eps)
        return ops.gemm(h, self.lm_head)

    # ---- DM / Generator ------------------------------------------------------------------
    def timestep_embedding(self, t: torch.Tensor) -> torch.Tensor:
        """t [B] in [0, 1] -> conditioning vector [B, d]."""
        e = sinusoidal_embedding(t, self.cfg.t_embed_dim).to(self.t_mlp1.dtype)
        h = F.silu(F.linear(e, self.t_mlp1, self.t_mlp1_b))
        return F.linear(h, self.t_mlp2, self.t_mlp2_b)

    def dm_embed(self, video_tokens: torch.Tensor, sound: Optional[torch.Tensor] = None,
                 action: Optional[torch.Tensor] = None, domain: int = 0, fps: Optional[int] = None,
                 cond_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """video_tokens [B, Sv, patch_dim] (+ sound [B, Ss, Cs], action [B, Sa, D<=action_dim_max])
        -> DM embeddings [B, Sv+Ss+Sa, d]. `cond_mask` [B, S] marks clean conditioning tokens."""
        dt = self.patch_in.dtype
        parts = [F.linear(video_tokens.to(dt), self.patch_in, self.patch_in_b)]
        if sound is not None:
            parts.append(F.linear(sound.to(dt), self.sound_in))
        if action is not None:
            a = F.pad(action.to(dt), (0, self.cfg.action_dim_max - action.shape[-1]))
            parts.append(F.linear(a, self.action_in[domain]))
        x = torch.cat(parts, dim=1) if len(parts) > 1 else parts[0]
        if fps is not None:
            x = x + self.fps_embed[min(int(fps), self.fps_embed.shape[0] - 1)]
        if cond_mask is not None:
            x = x + F.embedding(cond_mask.long(), self.cond_flag)
        return x

    def dm_forward(self, x: torch.Tensor, t: torch.Tensor, pos: torch.Tensor,
                   ar_kv: Optional[List[KV]] = None, ctx: AttnContext = LOCAL_ATTN,
                   layer_params: Optional[Callable] = None, checkpoint: bool = False,
                   cos_sin: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
        """x [B, S, d] DM embeddings, t [B], pos [3, S] -> hidden [B, S, d] (after final AdaLN norm)."""
        cfg = self.cfg
        cos, sin = cos_sin if cos_sin is not None else rope.rope_tables(pos, cfg.head_dim, cfg.rope_theta,
                                                                         cfg.mrope_section)
        t_emb = self.timestep_embedding(t)
        t_act = F.silu(t_emb)
        t_mod = F.linear(t_act, self.t_proj)
        for i, layer in enumerate(self.dm.layers):
            kv = None if ar_kv is None else ar_kv[i]
            if checkpoint and torch.is_grad_enabled():
                def run(x_, t_mod_, i=i, layer=layer, kv=kv):
                    p_ = layer.views() if layer_params is None else layer_params("dm", i)
                    return dm_block(cfg, p_, x_, t_mod_, cos, sin, kv, ctx)
                x = torch.utils.checkpoint.checkpoint(run, x, t_mod, use_reentrant=False)
            else:
                p = layer.views() if layer_params is None else layer_params("dm", i)
                x = dm_block(cfg, p, x, t_mod, cos, sin, kv, ctx)
        fm = F.linear(t_act, self.final_mod)
        d = cfg.d_model
        return ops.adaln_rmsnorm(x, self.dm_norm, fm[:, :d].contiguous(), fm[:, d:].contiguous(), x.shape[1],
                                 cfg.rms_eps)

    def dm_heads(self, hidden: torch.Tensor, n_video: int, n_sound: int = 0, n_action: int = 0,
                 domain: int = 0, action_dim: Optional[int] = None):
        """Splits the DM hidden states into per-modality velocity predictions."""
        out = {"video": F.linear(hidden[:, :n_video], self.patch_out)}
        off = n_video
        if n_sound:
            out["sound"] = F.linear(hidden[:, off:off + n_sound], self.sound_out)
            off += n_sound
        if n_action:
            a = F.linear(hidden[:, off:off + n_action], self.action_out[domain])
            out["action"] = a[..., :action_dim] if action_dim else a
        return out

    # ---- joint (training) ----------------------------------------------------------------
    def joint_forward(self, x_ar, pos_ar, x_dm, t, pos_dm, ctx: AttnContext = LOCAL_ATTN,
                      layer_params: Optional[Callable] = None, checkpoint: bool = False):
        cfg = self.cfg
        cos_a, sin_a = rope.rope_tables(pos_ar, cfg.head_dim, cfg.rope_theta, cfg.mrope_section)
        cos_d, sin_d = rope.rope_tables(pos_dm, cfg.head_dim, cfg.rope_theta, cfg.mrope_section)
        t_act = F.silu(self.timestep_embedding(t))
        t_mod = F.linear(t_act, self.t_proj)
        for i in range(cfg.n_layers):
            def run(xa, xd, tm, i=i):
                pa = self.ar.layers[i].views() if layer_params is None else layer_params("ar", i)
                pd = self.dm.layers[i].views() if layer_params is None else layer_params("dm", i)
                return joint_block(cfg, pa, pd, xa, xd, tm, cos_a, sin_a, cos_d, sin_d, ctx)
            if checkpoint and torch.is_grad_enabled():
                x_ar, x_dm = torch.utils.checkpoint.checkpoint(run, x_ar, x_dm, t_mod, use_reentrant=False)
            else:
                x_ar, x_dm = run(x_ar, x_dm, t_mod)
        fm = F.linear(t_act, self.final_mod)
        d = cfg.d_model
        h_dm = ops.adaln_rmsnorm(x_dm, self.dm_norm, fm[:, :d].contiguous(), fm[:, d:].contiguous(),
                                 x_dm.shape[1], cfg.rms_eps)
        return x_ar, h_dm


# --------------------------------------------------------------------------- patchify
def patchify(latent: torch.Tensor, cfg: MoTConfig) -> torch.Tensor:
    """[B, C, T, H, W] -> [B, T/pt * H/p * W/p, C*pt*p*p] (token order t, h, w)."""
    b, c, t, h, w = latent.shape
    pt, p = cfg.patch_t, cfg.patch_hw
    x = latent.reshape(b, c, t // pt, pt, h // p, p, w // p, p)
    x = x.permute(0, 2, 4, 6, 1, 3, 5, 7)
    return x.reshape(b, (t // pt) * (h // p) * (w // p), c * pt * p * p)


def unpatchify(tokens: torch.Tensor, cfg: MoTConfig, grid: Tuple[int, int, int]) -> torch.Tensor:
    """Inverse of `patchify`; grid = latent (T, H, W)."""
    b = tokens.shape[0]
    t, h, w = grid
    pt, p, c = cfg.patch_t, cfg.patch_hw, cfg.latent_channels
    x = tokens.reshape(b, t // pt, h // p, w // p, c, pt, p, p)
    x = x.permute(0, 4, 1, 5, 2, 6, 3, 7)
    return x.reshape(b, c, t, h, w)

"""Generator engine: prompt prefill on the AR tower, flow-matching denoise loop on the DM tower
with classifier-free guidance, and tokenizer decode.

The hot loop mirrors the reference's call stack (reference cookbooks/cosmos3/generator/
audiovisual/README.md:43-48 for the recipe; README.md:74 for the attention semantics):
for each step, run the DM tower on the cond and uncond branches (as one batch of 2, or one
branch per CFG-parallel rank), combine the velocities and advance the latent. The prompt's
AR-tower K/V are computed once and reused by all steps.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..config import MoTConfig, SamplingConfig
from . import rope, sampler as samplers
from .mot import KV, LOCAL_ATTN, AttnContext, MoTModel, WorkspaceAttn, patchify, unpatchify


@dataclass
class GenState:
    """Everything the denoise loop needs for one sample."""
    grid: Tuple[int, int, int]                 # latent (T, H, W)
    pos: torch.Tensor                          # [3, S_dm] positions of all DM tokens
    cos_sin: Tuple[torch.Tensor, torch.Tensor]
    ar_kv_cond: List[KV]
    ar_kv_uncond: Optional[List[KV]]
    n_video: int
    n_sound: int = 0
    n_action: int = 0
    domain: int = 0
    action_dim: Optional[int] = None
    fps: Optional[int] = None
    cond_mask: Optional[torch.Tensor] = None   # [S_dm] True = clean conditioning token (never updated)
    clean_tokens: Optional[torch.Tensor] = None  # [1, S_dm, F] values for the cond_mask positions
    # video transfer: clean latent tokens of the control clip (edge / blur / depth / seg / wsm map), [1, n_video, F] on
    # this rank's token shard. They run as a second vision stream that shares the target's 3-D rotary positions
    # (reference cookbooks/cosmos3/generator/transfer/README.md:35,98) and are flagged clean; `control_weight`
    # scales the control guidance term.
    control_tokens: Optional[torch.Tensor] = None
    control_weight: float = 1.0
    # context parallelism: this rank holds DM tokens [shard_start, shard_start + S_dm) of total_tokens
    shard_start: int = 0
    total_tokens: int = 0


class GeneratorEngine:
    def __init__(self, model: MoTModel, ctx: Optional[AttnContext] = None, cfg_group=None):
        """`ctx` is the attention/parallel context of the DM tower; `cfg_group` (optional) is a
        `parallel.cfgp.CFGParallel` that runs one guidance branch per rank group."""
        self.model = model
        self.cfg: MoTConfig = model.cfg
        dev = next(model.parameters()).device
        self.ctx = ctx if ctx is not None else (WorkspaceAttn() if dev.type == "cuda" else LOCAL_ATTN)
        self.cfg_group = cfg_group
        # Launch-bound steps (thumbnails, short low-resolution clips): the model evaluation of a denoise step is
        # captured in a CUDA graph once per generation and replayed for the other steps (the reference's PyTorch
        # engine also runs "with CUDA Graphs enabled where supported", inference_benchmarks.md:39). Sequences longer
        # than this many DM tokens run eagerly; 0 switches graphs off. Single-GPU layouts only
        # (COSMOS_CUDA_GRAPH_TOKENS). With this dense 8 B-parameter stand-in a 720p image (3600 tokens) and a
        # 61-frame 256p clip (7168 tokens) are already compute-bound at ~0.12 s per guided step: measured 4.29 s and
        # 4.41 s of sampling without a graph against 4.54 s and 4.68 s with one (the capture costs more than 35
        # replays save), hence the low default.
        import os
        self.graph_max_tokens = int(os.environ.get("COSMOS_CUDA_GRAPH_TOKENS", "1024"))

    # ------------------------------------------------------------------ prompt
    @torch.no_grad()
    def encode_prompt(self, ids: torch.Tensor) -> List[KV]:
        """ids [B, n] (already padded/truncated to the conditioning length) -> per-layer (K, V)."""
        pos = rope.text_positions(ids.shape[1], 0, ids.device)
        # a tensor-parallel model whose AR tower holds only this rank's heads runs the prompt through the same
        # rank group (all-reduced projections); every other layout runs the full AR tower locally
        pre = getattr(self.ctx, "prefill_context", None)
        if pre is not None and getattr(self.ctx, "presliced", False):
            _, kvs = self.model.ar_forward(self.model.embed_tokens(ids), pos, None, pre())
        else:
            _, kvs = self.model.ar_forward(self.model.embed_tokens(ids), pos)
        return kvs

    # ------------------------------------------------------------------ one DM evaluation
    @torch.no_grad()
    def velocity(self, tokens: torch.Tensor, sigma: torch.Tensor, st: GenState, ar_kv: List[KV],
                 with_control: bool = False) -> torch.Tensor:
        """tokens [B, S_dm, F] (noisy video/sound/action features, padded to a common width)
        -> velocity prediction of the same shape, bf16/fp32 as the model computes. `with_control` appends the
        state's control stream (clean tokens at the target's positions) to the sequence; its outputs are dropped."""
        if with_control:
            return self._velocity_with_control(tokens, sigma, st, ar_kv)
        m = self.model
        nv, ns, na = st.n_video, st.n_sound, st.n_action
        pd = self.cfg.patch_dim
        dt = m.patch_in.dtype
        video = tokens[:, :nv, :pd]
        sound = tokens[:, nv:nv + ns, :self.cfg.sound_latent_dim] if ns else None
        action = tokens[:, nv + ns:nv + ns + na, :st.action_dim] if na else None
        cm = None if st.cond_mask is None else st.cond_mask[None].expand(tokens.shape[0], -1)
        x = m.dm_embed(video.to(dt), sound, action, st.domain, st.fps, cm)
        h = m.dm_forward(x, sigma, st.pos, ar_kv, self.ctx, cos_sin=st.cos_sin)
        heads = m.dm_heads(h, nv, ns, na, st.domain, st.action_dim)
        out = torch.zeros(tokens.shape, dtype=heads["video"].dtype, device=tokens.device) \
            if (ns or na) else None
        if out is None:
            return heads["video"]
        out[:, :nv, :pd] = heads["video"]
        if ns:
            out[:, nv:nv + ns, :self.cfg.sound_latent_dim] = heads["sound"]
        if na:
            out[:, nv + ns:, :st.action_dim] = heads["action"]
        return out

    def _graphed_velocity(self, tokens: torch.Tensor, sigma: torch.Tensor, st: GenState, ar_kv: List[KV],
                          with_control: bool = False) -> torch.Tensor:
        """`velocity` through a CUDA graph when the call is small enough to be launch bound and runs on this GPU alone.
        The graph (inputs: tokens and sigma; everything else belongs to the generation state) is captured at the first
        call of a generation and kept on the state object; the result lives in the graph's static output buffer."""
        eligible = (tokens.is_cuda and self.graph_max_tokens > 0 and tokens.shape[1] <= self.graph_max_tokens
                    and self.cfg_group is None and type(self.ctx) in (AttnContext, WorkspaceAttn)
                    and tokens.dtype == torch.bfloat16 and ops.get_backend() == "own" and not torch.is_grad_enabled())
        if not eligible:
            return self.velocity(tokens, sigma, st, ar_kv, with_control)
        from ..utils.graphs import GraphedCallable
        graphs = st.__dict__.setdefault("_graphs", {})
        key = (tuple(tokens.shape), bool(with_control), id(ar_kv))
        if key not in graphs:
            graphs[key] = GraphedCallable(lambda t, s: self.velocity(t, s, st, ar_kv, with_control), [tokens, sigma])
        return graphs[key](tokens, sigma)

    @torch.no_grad()
    def _velocity_with_control(self, tokens, sigma, st: GenState, ar_kv: List[KV]) -> torch.Tensor:
        if st.n_sound or st.n_action:
            raise ValueError("a control stream needs a video-only token sequence")
        m, nv, pd = self.model, st.n_video, self.cfg.patch_dim
        dt = m.patch_in.dtype
        b = tokens.shape[0]
        ctrl = st.control_tokens[:, :, :pd].to(dt).expand(b, -1, -1)
        video = torch.cat([tokens[:, :nv, :pd].to(dt), ctrl], dim=1)
        cm = torch.zeros(b, 2 * nv, dtype=torch.bool, device=tokens.device)
        if st.cond_mask is not None:
            cm[:, :nv] = st.cond_mask[None, :nv]
        cm[:, nv:] = True
        x = m.dm_embed(video, None, None, st.domain, st.fps, cm)
        if not hasattr(st, "_ctrl_tables"):
            pos2 = torch.cat([st.pos[:, :nv], st.pos[:, :nv]], dim=1)
            st._ctrl_tables = (pos2, tuple(torch.cat([t[:nv], t[:nv]], dim=0) for t in st.cos_sin))
        pos2, cs2 = st._ctrl_tables
        h = m.dm_forward(x, sigma, pos2, ar_kv, self.ctx, cos_sin=cs2)
        return m.dm_heads(h[:, :nv], nv, 0, 0, st.domain, st.action_dim)["video"]

    def _control_scale(self, st: GenState, sc: SamplingConfig) -> float:
        """Weight of the control term v += w (v_ctrl - v_cond): the sampling's `control_guidance` (1 when a control
        clip is given without it) times the hint's `control_weight`; 0 without a control stream."""
        if st.control_tokens is None:
            return 0.0
        g = 1.0 if sc.control_guidance is None else float(sc.control_guidance)
        return g * float(st.control_weight)

    @torch.no_grad()
    def denoise_step(self, x: torch.Tensor, sigma: float, sigma_next: float, st: GenState,
                     sc: SamplingConfig, smp=None) -> torch.Tensor:
        """One guided step on the fp32 latent tokens x [1, S_dm, F]; returns the updated tokens."""
        dev = x.device
        use_cfg = (st.ar_kv_uncond is not None and sc.guidance != 1.0
                   and samplers.guidance_active(sigma, sc.guidance_interval))
        xin = x
        if st.cond_mask is not None and st.clean_tokens is not None:
            xin = torch.where(st.cond_mask[None, :, None], st.clean_tokens.to(x.dtype), x)
        mdt = self.model.patch_in.dtype
        gc = self._control_scale(st, sc)
        if self.cfg_group is not None and use_cfg:
            vc, vu = self.cfg_group.branch_velocities(self, xin, sigma, st, control_scale=gc,
                                                      guidance=sc.guidance)
            gc = 0.0   # already folded into the cond branch
        elif use_cfg:
            kv2 = [(torch.cat([kc, ku]), torch.cat([vc_, vu_]))
                   for (kc, vc_), (ku, vu_) in zip(st.ar_kv_cond, st.ar_kv_uncond)] \
                if not hasattr(st, "_kv2") else st._kv2
            st._kv2 = kv2
            sig = torch.full((2,), float(sigma), device=dev)
            v2 = self._graphed_velocity(xin.to(mdt).expand(2, -1, -1).contiguous(), sig, st, kv2)
            vc, vu = v2[:1], v2[1:]
        else:
            sig = torch.full((1,), float(sigma), device=dev)
            vc, vu = self._graphed_velocity(xin.to(mdt), sig, st, st.ar_kv_cond), None
        if gc != 0.0:
            # third branch: the same prompt with the control stream. v = v_u + g (v_c - v_u) + g_c (v_ctrl - v_c)
            # equals the two-branch formula with v_c replaced by v_c + (g_c / g) (v_ctrl - v_c), so the fused
            # CFG + sampler kernel serves it unchanged.
            sig1 = torch.full((1,), float(sigma), device=dev)
            v_ctrl = self._graphed_velocity(xin.to(mdt), sig1, st, st.ar_kv_cond, with_control=True)
            w = gc / float(sc.guidance) if vu is not None else gc
            vc = torch.lerp(vc.float(), v_ctrl.float(), w).to(vc.dtype)
        if smp is None or isinstance(smp, samplers.EulerSampler):
            dt = float(sigma_next - sigma)
            if smp is not None:
                smp.i += 1
            s, f = x.shape[1], x.shape[2]
            x2 = x.reshape(s, f)
            if x2.is_cuda and vc.dtype == torch.bfloat16:
                x_new = ops.cfg_euler_step(x2.contiguous(), vc.reshape(s, f), None if vu is None else vu.reshape(s, f),
                                           sc.guidance, dt, sc.normalize_cfg).reshape(x.shape)
            else:
                x_new = ops.ref.cfg_euler_step(x2, vc.reshape(s, f), None if vu is None else vu.reshape(s, f),
                                               sc.guidance, dt, sc.normalize_cfg).reshape(x.shape).to(x.dtype)
        elif isinstance(smp, samplers.UniPCSampler) and x.is_cuda and vc.dtype == torch.bfloat16 and x.shape[0] == 1:
            s, f = x.shape[1], x.shape[2]
            x_new = ops.cfg_unipc_step(x.reshape(s, f).contiguous(), vc.reshape(s, f),
                                       None if vu is None else vu.reshape(s, f), sc.guidance, smp,
                                       sc.normalize_cfg).reshape(x.shape)
        else:
            v = samplers.cfg_velocity(vc, vu, sc.guidance, sc.normalize_cfg)
            x_new = smp.step(x, v.to(x.dtype))
        if st.cond_mask is not None and st.clean_tokens is not None:
            x_new = torch.where(st.cond_mask[None, :, None], st.clean_tokens.to(x_new.dtype), x_new)
        return x_new

    # ------------------------------------------------------------------ full loop
    @torch.no_grad()
    def sample(self, st: GenState, sc: SamplingConfig, noise: Optional[torch.Tensor] = None,
               feat_dim: Optional[int] = None, callback=None) -> torch.Tensor:
        """Runs the whole denoise loop and returns the final fp32 tokens [1, S_dm, F]."""
        dev = st.pos.device
        s_dm = st.pos.shape[1]
        f = feat_dim or self.cfg.patch_dim
        if noise is None:
            g = torch.Generator(device=dev)
            g.manual_seed(sc.seed)
            noise = torch.randn(1, s_dm, f, generator=g, device=dev, dtype=torch.float32)
        sig = samplers.shifted_sigmas(sc.num_steps, sc.shift, sc.sigma_max, device="cpu")
        smp = samplers.make_sampler(sc.scheduler, sig)
        x = noise.float() * float(sig[0]) if sc.sigma_max is not None else noise.float()
        for i in range(sc.num_steps):
            x = self.denoise_step(x, float(sig[i]), float(sig[i + 1]), st, sc, smp)
            if callback is not None:
                callback(i, x)
        return x

    def make_state(self, ids_cond: torch.Tensor, ids_uncond: Optional[torch.Tensor],
                   grid: Tuple[int, int, int], n_sound: int = 0, n_action: int = 0, **kw) -> GenState:
        cfg = self.cfg
        dev = ids_cond.device
        tgrid = (grid[0] // cfg.patch_t, grid[1] // cfg.patch_hw, grid[2] // cfg.patch_hw)
        pp = rope.generator_positions(ids_cond.shape[1], tgrid, n_sound, n_action, dev)
        parts = [pp["video"]] + ([pp["sound"]] if n_sound else []) + ([pp["action"]] if n_action else [])
        pos = torch.cat(parts, dim=1)
        total = pos.shape[1]
        n_video, start = pp["video"].shape[1], 0
        cp, cp_rank = getattr(self.ctx, "cp", 1), getattr(self.ctx, "rank", 0)
        if cp > 1:
            if n_sound or n_action or total % cp:
                raise ValueError("context parallelism needs a video-only token sequence divisible by cp")
            n_video = total // cp
            start = cp_rank * n_video
            pos = pos[:, start:start + n_video].contiguous()
        cos_sin = rope.rope_tables(pos, cfg.head_dim, cfg.rope_theta, cfg.mrope_section)
        kv_c = self.encode_prompt(ids_cond)
        kv_u = self.encode_prompt(ids_uncond) if ids_uncond is not None else None
        return GenState(grid=grid, pos=pos, cos_sin=cos_sin, ar_kv_cond=kv_c, ar_kv_uncond=kv_u,
                        n_video=n_video, n_sound=n_sound, n_action=n_action, shard_start=start,
                        total_tokens=total, **kw)

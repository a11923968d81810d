"""Vision encoder of the Reasoner (AR side): a ViT over 16x16 patches with temporal patch 2 and
2x2 spatial merge, producing one d_model embedding per merged patch (Qwen3-VL conventions, which
the reference's Reasoner follows: reference README.md:145,286 and
cookbooks/cosmos3/reasoner/reasoner_prompt_guide.md:77-99): learned position table sampled bilinearly, 2-D rotary
embedding in every block, attention within a temporal slice, LayerNorm + two-layer merger over each 2x2 block.
With the weights of a Qwen3-VL vision tower mapped in (ckpt/hf_qwen3vl.py) the outputs agree with the
`transformers` implementation (tests/test_hf_parity_cpu.py). With `cfg.vit_deepstack` the features
after the listed blocks go through mergers of their own and are handed to the language tower, which
adds them to the hidden states of its first layers at the vision positions (DeepStack)."""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import MoTConfig


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    a, b = x.chunk(2, dim=-1)
    return torch.cat([-b, a], dim=-1)


def rotary_2d(gh: int, gw: int, head_dim: int, device, theta: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [gh * gw, head_dim] of the 2-D rotary embedding of the vision blocks: a quarter of the head
    dimension's frequencies turn with the patch row, the next quarter with the patch column, and that half is
    repeated for the second half of the head (Qwen3-VL vision convention, `transformers`
    models/qwen3_vl/modeling_qwen3_vl.py, `rot_pos_emb`)."""
    quarter = head_dim // 4
    inv = 1.0 / (theta ** (torch.arange(0, 2 * quarter, 2, dtype=torch.float32, device=device) / (2 * quarter)))
    rows = torch.arange(gh, device=device, dtype=torch.float32)[:, None, None].expand(gh, gw, 1) * inv
    cols = torch.arange(gw, device=device, dtype=torch.float32)[None, :, None].expand(gh, gw, 1) * inv
    ang = torch.cat([rows, cols], dim=-1).reshape(gh * gw, 2 * quarter)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


class ViTBlock(nn.Module):
    def __init__(self, dim: int, heads: int, ffn: int = 0):
        super().__init__()
        self.heads = heads
        ffn = ffn or 4 * dim
        self.n1, self.n2 = nn.LayerNorm(dim, eps=1e-6), nn.LayerNorm(dim, eps=1e-6)
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.fc1, self.fc2 = nn.Linear(dim, ffn), nn.Linear(ffn, dim)

    def forward(self, x, rot=None):
        b, s, d = x.shape
        q, k, v = self.qkv(self.n1(x)).view(b, s, 3, self.heads, d // self.heads).unbind(2)
        if rot is not None:  # cos / sin [s, head_dim], the same for every temporal slice
            cos, sin = rot[0][None, :, None], rot[1][None, :, None]
            q = (q.float() * cos + _rotate_half(q.float()) * sin).to(x.dtype)
            k = (k.float() * cos + _rotate_half(k.float()) * sin).to(x.dtype)
        # attention within a temporal slice; the library's fused kernel keeps memory linear in the patch count
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        o = o.transpose(1, 2).reshape(b, s, d)
        x = x + self.proj(o)
        return x + self.fc2(F.gelu(self.fc1(self.n2(x)), approximate="tanh"))


class VisionEncoder(nn.Module):
    def __init__(self, cfg: MoTConfig):
        super().__init__()
        self.cfg = cfg
        p, tp, hdim = cfg.vit_patch, cfg.vit_temporal_patch, cfg.vit_hidden
        self.patch = nn.Linear(3 * tp * p * p, hdim)
        self.pos_side = cfg.vit_pos_side
        self.pos = nn.Parameter(torch.zeros(self.pos_side * self.pos_side, hdim))
        self.blocks = nn.ModuleList([ViTBlock(hdim, cfg.vit_heads, cfg.vit_ffn) for _ in range(cfg.vit_depth)])
        self.norm = nn.LayerNorm(hdim, eps=1e-6)
        m = cfg.vit_spatial_merge
        self.merge = nn.Sequential(nn.Linear(hdim * m * m, hdim * m * m), nn.GELU(), nn.Linear(hdim * m * m, cfg.d_model))
        self.deepstack = tuple(i for i in cfg.vit_deepstack if 0 <= i < cfg.vit_depth)
        self.deepstack_norm = nn.ModuleList([nn.LayerNorm(hdim * m * m, eps=1e-6) for _ in self.deepstack])
        self.deepstack_merge = nn.ModuleList([
            nn.Sequential(nn.Linear(hdim * m * m, hdim * m * m), nn.GELU(), nn.Linear(hdim * m * m, cfg.d_model))
            for _ in self.deepstack])
        nn.init.normal_(self.pos, std=0.02)

    def grid(self, frames: int, height: int, width: int) -> Tuple[int, int, int]:
        """Token grid (t, h, w) after temporal patching and spatial merge."""
        c = self.cfg
        t = max(1, (frames + c.vit_temporal_patch - 1) // c.vit_temporal_patch)
        unit = c.vit_patch * c.vit_spatial_merge
        return t, height // unit, width // unit

    def forward(self, video: torch.Tensor, return_deepstack: bool = False):
        """video [T, 3, H, W] in [-1, 1] (H, W multiples of patch*merge) -> ([t*h*w, d_model], (t, h, w))
        and, with `return_deepstack`, the list of DeepStack features [t*h*w, d_model] (one per listed block)."""
        c = self.cfg
        p, tp, m = c.vit_patch, c.vit_temporal_patch, c.vit_spatial_merge
        t_in, _, hh, ww = video.shape
        if t_in % tp:
            video = torch.cat([video, video[-1:].expand(tp - t_in % tp, -1, -1, -1)])
        t = video.shape[0] // tp
        gh, gw = hh // p, ww // p
        x = video.view(t, tp, 3, gh, p, gw, p).permute(0, 3, 5, 2, 1, 4, 6).reshape(t, gh * gw, -1)
        x = self.patch(x.to(self.patch.weight.dtype))
        # the learned table is sampled bilinearly on a grid whose corners coincide with the table's corners
        side = self.pos_side
        pos = F.interpolate(self.pos.view(1, side, side, -1).permute(0, 3, 1, 2).float(), size=(gh, gw), mode="bilinear",
                            align_corners=True).permute(0, 2, 3, 1).reshape(1, gh * gw, -1).to(x.dtype)
        x = x + pos
        rot = rotary_2d(gh, gw, c.vit_hidden // c.vit_heads, x.device)
        def merged(y):  # [t, gh * gw, hidden] -> [t * (gh/m) * (gw/m), hidden * m * m]
            y = y.view(t, gh // m, m, gw // m, m, -1).permute(0, 1, 3, 2, 4, 5)
            return y.reshape(t * (gh // m) * (gw // m), -1)

        deep: List[torch.Tensor] = []
        for i, blk in enumerate(self.blocks):  # attention within each temporal slice
            x = blk(x, rot)
            if i in self.deepstack:
                k = self.deepstack.index(i)
                deep.append(self.deepstack_merge[k](self.deepstack_norm[k](merged(x))))
        out = self.merge(merged(self.norm(x)))
        grid = (t, gh // m, gw // m)
        if return_deepstack:
            return out, grid, deep
        return out, grid

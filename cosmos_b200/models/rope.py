"""3D multimodal rotary position ids and cos/sin tables (interleaved mRoPE).

Every token carries (t, h, w) position ids. Text tokens use the same running index on all
three axes; a vision block starting at running index p0 uses (p0 + frame, p0 + row, p0 + col),
and the running index then jumps past the block's largest id (Qwen3-VL convention; the
reference states "3D mRoPE" across image, video, audio and action tokens, README.md:74).
Frequencies are assigned to axes in the interleaved pattern T,H,W,T,H,W,... for the first
3*min(section) indices and the rest to T, which is what `mrope_section=[24,20,20]` means for
head_dim 128.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch


def axis_of_frequency(half_dim: int, section: Sequence[int]) -> torch.Tensor:
    """For each of the half_dim rotary frequencies: which axis (0=t, 1=h, 2=w) drives it."""
    st, sh, sw = section
    assert st + sh + sw == half_dim, f"mrope_section {section} must sum to {half_dim}"
    axis = torch.zeros(half_dim, dtype=torch.long)
    axis[1:sh * 3:3] = 1
    axis[2:sw * 3:3] = 2
    return axis


def rope_tables(pos: torch.Tensor, head_dim: int, theta: float, section: Sequence[int]
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """pos [3, S] (t, h, w) -> cos, sin [S, head_dim/2] fp32 (rotate-half convention)."""
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64, device=pos.device) * 2.0 / head_dim))
    axis = axis_of_frequency(half, section).to(pos.device)
    p = pos.to(torch.float64)[axis, :]            # [half, S]
    ang = (p * inv_freq[:, None]).t().contiguous()  # [S, half]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def text_positions(n: int, start: int = 0, device=None) -> torch.Tensor:
    idx = torch.arange(start, start + n, device=device)
    return idx[None, :].expand(3, -1).contiguous()


def grid_positions(t: int, h: int, w: int, start: int = 0, device=None, t_scale: float = 1.0) -> torch.Tensor:
    """[3, t*h*w] ids of a (t, h, w) token grid in row-major (t, h, w) order."""
    tt = (torch.arange(t, device=device).float() * t_scale).round().long()
    ti = tt[:, None, None].expand(t, h, w)
    hi = torch.arange(h, device=device)[None, :, None].expand(t, h, w)
    wi = torch.arange(w, device=device)[None, None, :].expand(t, h, w)
    return torch.stack([ti, hi, wi]).reshape(3, -1) + start


def next_start(pos: torch.Tensor) -> int:
    """Running index after a block: one past its largest id."""
    return int(pos.max().item()) + 1 if pos.numel() else 0


def generator_positions(n_text: int, grid: Tuple[int, int, int], n_sound: int = 0, n_action: int = 0,
                        device=None, share_temporal_with: Optional[torch.Tensor] = None,
                        n_control: int = 0):
    """Position ids of a Generator sequence: text | video grid | [control grid] | sound | action.

    Sound and action tokens are temporal streams: they advance along t only and sit at h = w = 0
    of the video block, so that token i of either stream is aligned in time with the video.
    With `n_control` > 0 a second grid (the transfer control video) follows the target grid and,
    when `share_temporal_with` is given, reuses the target's temporal ids
    (`share_vision_temporal_positions` in the reference's transfer specs, specs/edge.json:14).
    """
    out = {}
    p_text = text_positions(n_text, 0, device)
    start = n_text
    t, h, w = grid
    p_vid = grid_positions(t, h, w, start, device)
    out["text"], out["video"] = p_text, p_vid
    after = next_start(p_vid) if p_vid.numel() else start
    if n_control:
        p_ctl = grid_positions(t, h, w, start if share_temporal_with is not None else after, device)
        out["control"] = p_ctl
        after = max(after, next_start(p_ctl))
    if n_sound:
        ts = torch.linspace(0, max(t - 1, 0), n_sound, device=device).round().long() + start
        out["sound"] = torch.stack([ts, torch.full_like(ts, start), torch.full_like(ts, start)])
    if n_action:
        ta = torch.linspace(0, max(t - 1, 0), n_action, device=device).round().long() + start
        out["action"] = torch.stack([ta, torch.full_like(ta, start), torch.full_like(ta, start)])
    return out

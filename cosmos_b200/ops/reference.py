"""Plain-PyTorch definitions of every fused op.

They serve three purposes: the CPU execution path (tests, gloo plumbing), the numerics
oracle for the CUDA kernels (computed in fp32), and the statement of each op's contract.
All functions compute in fp32 and cast the result back to the input dtype.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

EPI_PLAIN, EPI_SWIGLU, EPI_GATED_RESID, EPI_QKV_ROPE = 0, 1, 2, 3
MASK_FULL, MASK_CAUSAL, MASK_MOT = 0, 1, 2


def _rows_to_batch(t: torch.Tensor, rows: int, rows_per_batch: int) -> torch.Tensor:
    """Expands a per-batch [B, d] modulation tensor to one row per token."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.shape[0] == 1:
        return t2.expand(rows, -1)
    idx = torch.arange(rows, device=t.device) // rows_per_batch
    return t2[idx]


def rmsnorm(x, gamma=None, eps: float = 1e-6, residual=None):
    xf = x.float()
    res_out = None
    if residual is not None:
        xf = xf + residual.float()
        res_out = xf.to(x.dtype)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if gamma is not None:
        y = y * gamma.float()
    return y.to(x.dtype), res_out


def adaln_rmsnorm(x, gamma, shift, scale, rows_per_batch: int, eps: float = 1e-6):
    d = x.shape[-1]
    xf = x.float().reshape(-1, d)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if gamma is not None:
        y = y * gamma.float()
    sh = _rows_to_batch(shift, xf.shape[0], rows_per_batch).float()
    sc = _rows_to_batch(scale, xf.shape[0], rows_per_batch).float()
    y = y * (1.0 + sc) + sh
    return y.to(x.dtype).reshape(x.shape)


def rotate_half_apply(x, cos, sin):
    """x [..., rows, heads, D]; cos/sin [rows, D/2] (rotate-half convention)."""
    d2 = x.shape[-1] // 2
    xf = x.float()
    a, b = xf[..., :d2], xf[..., d2:]
    rows = x.shape[-3]
    rr = cos.shape[0]
    if rr != rows:
        idx = torch.arange(rows, device=x.device) % rr
        cos, sin = cos[idx], sin[idx]
    c = cos.float()[:, None, :]
    s = sin.float()[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def mrope(x, cos=None, sin=None, gamma=None, eps: float = 1e-6):
    """Per-head RMSNorm (optional) followed by rotary embedding (optional); x [.., rows, H, D]."""
    xf = x.float()
    if gamma is not None:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    if cos is not None:
        shp = xf.shape
        x3 = xf.reshape(-1, shp[-2], shp[-1])
        xf = rotate_half_apply(x3, cos, sin).reshape(shp)
    return xf.to(x.dtype)


def gated_residual(x, f, gate=None, rows_per_batch: int = 1):
    d = x.shape[-1]
    xf = x.float().reshape(-1, d)
    ff = f.float().reshape(-1, d)
    if gate is not None:
        ff = ff * _rows_to_batch(gate, xf.shape[0], rows_per_batch).float()
    return (xf + ff).to(x.dtype).reshape(x.shape)


def swiglu(gate_up):
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def gemm(a, w, bias=None, epi: int = EPI_PLAIN, resid=None, gate=None, rows_per_batch: int = 0):
    acc = a.float() @ w.float().t()
    if bias is not None:
        acc = acc + bias.float()
    if epi == EPI_SWIGLU:
        g, u = acc.chunk(2, dim=-1)
        acc = F.silu(g) * u
    elif epi == EPI_GATED_RESID:
        n = acc.shape[-1]
        flat = acc.reshape(-1, n)
        if gate is not None:
            flat = flat * _rows_to_batch(gate, flat.shape[0], rows_per_batch).float()
        acc = (resid.float().reshape(-1, n) + flat).reshape(acc.shape)
    return acc.to(a.dtype)


def gemm_qkv_rope(a, w, bias, cos, sin, gamma_q, gamma_k, n_q_heads: int, n_k_heads: int, eps: float = 1e-6):
    """QKV projection + per-head q/k RMSNorm + rotary embedding. Returns [..., N]."""
    acc = a.float() @ w.float().t()
    if bias is not None:
        acc = acc + bias.float()
    lead = acc.shape[:-1]
    n = acc.shape[-1]
    h = acc.reshape(-1, n // 128, 128)
    q = h[:, :n_q_heads]
    k = h[:, n_q_heads:n_q_heads + n_k_heads]
    v = h[:, n_q_heads + n_k_heads:]
    q = mrope(q, cos, sin, gamma_q, eps)
    k = mrope(k, cos, sin, gamma_k, eps)
    return torch.cat([q, k, v], dim=1).reshape(*lead, n).to(a.dtype)


def attention_mask(sq: int, skv: int, mask: int, n_ar: int = 0, device=None) -> Optional[torch.Tensor]:
    """Boolean [sq, skv] mask (True = attend) for the three mask modes."""
    if mask == MASK_FULL:
        return None
    qi = torch.arange(sq, device=device)[:, None]
    kj = torch.arange(skv, device=device)[None, :]
    if mask == MASK_CAUSAL:
        return kj <= qi + (skv - sq)
    if mask == MASK_MOT:
        ar_row = qi < n_ar
        return torch.where(ar_row, kj <= qi, torch.ones_like(kj, dtype=torch.bool))
    raise ValueError(f"unknown mask {mask}")


def attention(q, k, v, scale: Optional[float] = None, mask: int = MASK_FULL, n_ar: int = 0,
              return_lse: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q [B, Sq, Hq, D]; k, v [B, Skv, Hkv, D] -> o [B, Sq, Hq, D], lse [B, Hq, Sq] (natural log)."""
    b, sq, hq, d = q.shape
    skv, hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(hq // hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(hq // hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    m = attention_mask(sq, skv, mask, n_ar, q.device)
    if m is not None:
        s = s.masked_fill(~m, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), (lse if return_lse else None)


def cfg_combine(vc, vu, guidance: float, normalize: bool = False):
    """v = vu + g (vc - vu); with `normalize`, rows are rescaled so |v| <= |vc| (row = last dim)."""
    c = vc.float()
    if vu is None:
        return c
    v = vu.float() + guidance * (c - vu.float())
    if normalize:
        nc = c.pow(2).sum(-1, keepdim=True)
        nv = v.pow(2).sum(-1, keepdim=True)
        rs = torch.where(nv > 0, torch.sqrt(nc / nv.clamp_min(1e-30)).clamp(max=1.0), torch.ones_like(nv))
        v = v * rs
    return v


def cfg_euler_step(x, vc, vu, guidance: float, dt: float, normalize: bool = False):
    """x (fp32) + dt * cfg(vc, vu); returns the new latent (fp32)."""
    v = cfg_combine(vc.reshape(x.shape), None if vu is None else vu.reshape(x.shape), guidance, normalize)
    return x.float() + dt * v

"""The same ops on PyTorch's library kernels (cuBLAS matmul, fused SDPA, eager element-wise), in the input dtype.

This is the comparison arm, not a fallback: `ops.set_backend("library")` (or COSMOS_OPS_BACKEND=library)
routes every op here, so that the identical model, layout and sampler can be timed on library kernels with
NCCL collectives (`bench.py --impl library`). The reference publishes its numbers for such a build
("PyTorch" engine, inference_benchmarks.md:39,130-133). Results differ from the hand-written kernels only by
rounding (intermediate tensors are rounded to bf16 where a fused kernel keeps fp32 in registers).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .reference import (EPI_GATED_RESID, EPI_PLAIN, EPI_SWIGLU, MASK_CAUSAL, MASK_FULL, MASK_MOT, _rows_to_batch,
                        attention_mask)


def _norm(x, gamma, eps):
    return F.rms_norm(x, (x.shape[-1],), gamma, eps)


def rmsnorm(x, gamma=None, eps: float = 1e-6, residual=None):
    res_out = None
    if residual is not None:
        x = x + residual
        res_out = x
    return _norm(x, gamma, eps), res_out


def adaln_rmsnorm(x, gamma, shift, scale, rows_per_batch: int, eps: float = 1e-6):
    d = x.shape[-1]
    y = _norm(x.reshape(-1, d), gamma, eps)
    sh = _rows_to_batch(shift, y.shape[0], rows_per_batch)
    sc = _rows_to_batch(scale, y.shape[0], rows_per_batch)
    return torch.addcmul(sh, y, 1.0 + sc).reshape(x.shape)


def _rotate(x, cos, sin):
    """x [rows, H, D]; cos/sin [rr, D/2]; rows % rr == 0."""
    d2 = x.shape[-1] // 2
    rows, rr = x.shape[0], cos.shape[0]
    if rr != rows:
        idx = torch.arange(rows, device=x.device) % rr
        cos, sin = cos[idx], sin[idx]
    c = cos.to(x.dtype)[:, None, :]
    s = sin.to(x.dtype)[:, None, :]
    a, b = x[..., :d2], x[..., d2:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def mrope(x, cos=None, sin=None, gamma=None, eps: float = 1e-6):
    if gamma is not None:
        x = _norm(x, gamma, eps)
    if cos is not None:
        shp = x.shape
        x = _rotate(x.reshape(-1, shp[-2], shp[-1]), cos, sin).reshape(shp)
    return x


def gated_residual(x, f, gate=None, rows_per_batch: int = 1):
    d = x.shape[-1]
    if gate is None:
        return x + f
    g = _rows_to_batch(gate, x.numel() // d, rows_per_batch)
    return torch.addcmul(x.reshape(-1, d), f.reshape(-1, d), g).reshape(x.shape)


def swiglu(gate_up):
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


def gemm(a, w, bias=None, epi: int = EPI_PLAIN, resid=None, gate=None, rows_per_batch: int = 0):
    acc = F.linear(a, w, bias)
    if epi == EPI_SWIGLU:
        return swiglu(acc)
    if epi == EPI_GATED_RESID:
        return gated_residual(resid.reshape(acc.shape), acc, gate, rows_per_batch)
    return acc


def gemm_qkv_rope(a, w, bias, cos, sin, gamma_q, gamma_k, n_q_heads: int, n_k_heads: int, eps: float = 1e-6):
    acc = F.linear(a, w, bias)
    lead, n = acc.shape[:-1], acc.shape[-1]
    h = acc.reshape(-1, n // 128, 128)
    q = mrope(h[:, :n_q_heads], cos, sin, gamma_q, eps)
    k = mrope(h[:, n_q_heads:n_q_heads + n_k_heads], cos, sin, gamma_k, eps)
    return torch.cat([q, k, h[:, n_q_heads + n_k_heads:]], dim=1).reshape(*lead, n)


def attention(q, k, v, scale: Optional[float] = None, mask: int = MASK_FULL, n_ar: int = 0,
              return_lse: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """SDPA on [B, H, S, D] views (fused kernel of the library: cuDNN / flash); GQA through `enable_gqa`."""
    b, sq, hq, d = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    if return_lse:
        from . import reference as ref
        return ref.attention(q, k, v, scale, mask, n_ar, True)
    if mask == MASK_FULL:
        o = F.scaled_dot_product_attention(qt, kt, vt, scale=scale, enable_gqa=True)
    elif mask == MASK_CAUSAL and sq == k.shape[1]:
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, scale=scale, enable_gqa=True)
    else:
        m = attention_mask(sq, k.shape[1], mask, n_ar, q.device)
        o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=m, scale=scale, enable_gqa=True)
    return o.permute(0, 2, 1, 3), None


def cfg_euler_step(x, vc, vu, guidance: float, dt: float, normalize: bool = False):
    from .reference import cfg_combine
    v = cfg_combine(vc.reshape(x.shape), None if vu is None else vu.reshape(x.shape), guidance, normalize)
    return x.float() + dt * v

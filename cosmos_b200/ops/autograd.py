"""Autograd functions whose forward AND backward tensor-core work runs on this package's sm_100a
kernels (training path on CUDA bf16):

  linear     fwd  y = x W^T                      tcgen05 GEMM
             bwd  dX = dY W, dW = dY^T X         the same kernel reading the transposed operands in
                                                 place (MN-major shared-memory tiles)
  attention  fwd  flash attention (tcgen05) with the log-sum-exp saved
             bwd  flash backward on tcgen05 (csrc/attn_bwd_tcgen05.cu): a dK/dV kernel with the K/V
                  tile stationary and a dQ kernel with the Q tile stationary; scores are recomputed
                  on chip, nothing of size S^2 reaches memory.
                  COSMOS_ATTN_BWD_MATERIALIZED=1 selects the older per-head variant with scores
                  materialised as bf16 [Sq, Skv]:
                  P  = exp(Q K^T scale - lse)    GEMM with the exp in its epilogue (fp32 scores never leave TMEM)
                  dS = P (dO V^T - D) scale      GEMM with P as an epilogue operand
                  dV = P^T dO, dQ = dS K, dK = dS^T Q   plain GEMMs on transposed operands
                  This moves O(S^2) bytes per head instead of recomputing tiles on chip, which is
                  about 2x the cost of a fused flash backward at the 14k-token training shapes and
                  keeps every FLOP on this package's kernels.
Element-wise pieces of the layer (norms, SwiGLU, rotary, residuals) use PyTorch autograd.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .reference import MASK_CAUSAL, MASK_FULL, MASK_MOT


def _k():
    return torch.ops.cosmos_b200


_MATERIALIZED = os.environ.get("COSMOS_ATTN_BWD_MATERIALIZED", "0") == "1"


class LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        y = _k().gemm(x2, w, None, 0, None, None, 0, None)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1 or dy2.stride(0) % 8 != 0:
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = _k().gemm_ex(dy2, w, False, True, None).reshape(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = _k().gemm_ex(dy2, x2, True, True, None)
        return dx, dw


def linear(x, w):
    return LinearFn.apply(x, w)


class AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, mask, n_ar):
        o, lse = _k().attn_fwd(q, k, v, scale, mask, n_ar, True, None, 0, None)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.mask, ctx.n_ar = scale, mask, n_ar
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        scale, mask, n_ar = ctx.scale, ctx.mask, ctx.n_ar
        b, sq, hq, d = q.shape
        skv, hkv = k.shape[1], k.shape[2]
        group = hq // hkv
        do = do.contiguous()
        if not _MATERIALIZED:
            delta = (do.float() * o.float()).sum(-1).permute(0, 2, 1).contiguous()  # [B, Hq, Sq]
            dq, dk, dv = _k().attn_bwd(q, k, v, do, lse, delta, scale, mask, n_ar)
            return dq, dk, dv, None, None, None
        dq = torch.empty_like(q)
        dk = torch.zeros(b, skv, hkv, d, dtype=torch.float32, device=q.device)
        dv = torch.zeros_like(dk)
        delta = (do.float() * o.float()).sum(-1).permute(0, 2, 1).contiguous()  # [B, Hq, Sq]
        ld = (skv + 7) // 8 * 8
        p_buf = torch.empty(sq, ld, dtype=q.dtype, device=q.device)[:, :skv]
        ds_buf = torch.empty(sq, ld, dtype=q.dtype, device=q.device)[:, :skv]
        for bi in range(b):
            for h in range(hq):
                kh = h // group
                qh, kh_, vh, doh = q[bi, :, h], k[bi, :, kh], v[bi, :, kh], do[bi, :, h]
                _k().attn_bwd_scores(qh, kh_, lse[bi, h].contiguous(), scale, mask, n_ar, 0, None, p_buf)
                _k().attn_bwd_scores(doh, vh, delta[bi, h], scale, mask, n_ar, 1, p_buf, ds_buf)
                dv[bi, :, kh] += _k().gemm_ex(p_buf, doh, True, True, None).float()
                dk[bi, :, kh] += _k().gemm_ex(ds_buf, qh, True, True, None).float()
                dq[bi, :, h] = _k().gemm_ex(ds_buf, kh_, False, True, None)
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None


def attention(q, k, v, scale: Optional[float] = None, mask: int = MASK_FULL, n_ar: int = 0):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return AttentionFn.apply(q, k, v, float(scale), int(mask), int(n_ar))

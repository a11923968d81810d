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
  norms, q/k norm + rotary, SwiGLU, gated residual: forward kernels of csrc/elementwise.cu,
             backward kernels of csrc/elementwise_bwd.cu (row gradients in one pass; the gradients of
             gamma / shift / scale / gate as per-block partial sums, summed here).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .reference import MASK_FULL, MASK_MOT


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


# --------------------------------------------------------------------------- bandwidth pieces
def _sum_to(t: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """Per-batch sums [B, d] -> the shape of the input they belong to ([B, d], [1, d] or [d])."""
    if like.numel() == t.shape[-1]:
        t = t.sum(0)
    return t.reshape(like.shape).to(like.dtype)


class AdaLNRMSNormFn(torch.autograd.Function):
    """y = rmsnorm(x) * gamma * (1 + scale[b]) + shift[b]; forward and backward on the sm_100a kernels
    (csrc/elementwise.cu, csrc/elementwise_bwd.cu)."""

    @staticmethod
    def forward(ctx, x, gamma, shift, scale, rows_per_batch, eps):
        xc = x.contiguous()
        ctx.save_for_backward(xc, gamma, shift, scale)
        ctx.rpb, ctx.eps = int(rows_per_batch), float(eps)
        return _k().adaln_rmsnorm(xc, gamma, shift, scale, rows_per_batch, eps)

    @staticmethod
    def backward(ctx, dy):
        x, gamma, shift, scale = ctx.saved_tensors
        dx, part = _k().rmsnorm_bwd(x, dy.contiguous(), gamma, scale, ctx.rpb, ctx.eps, True)
        sums = part.sum(1)  # [B, 3, d]
        dgamma = sums[:, 2].sum(0).to(gamma.dtype) if (gamma is not None and ctx.needs_input_grad[1]) else None
        dshift = _sum_to(sums[:, 0], shift) if ctx.needs_input_grad[2] else None
        dscale = _sum_to(sums[:, 1], scale) if ctx.needs_input_grad[3] else None
        return dx, dgamma, dshift, dscale, None, None


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, eps):
        xc = x.contiguous()
        ctx.save_for_backward(xc, gamma)
        ctx.eps = float(eps)
        y, _ = _k().rmsnorm(xc, gamma, eps, None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma = ctx.saved_tensors
        want = gamma is not None and ctx.needs_input_grad[1]
        dx, part = _k().rmsnorm_bwd(x, dy.contiguous(), gamma, None, 0, ctx.eps, want)
        dgamma = part.sum((0, 1))[2].to(gamma.dtype) if want else None
        return dx, dgamma, None


class QKVPostFn(torch.autograd.Function):
    """qkv [rows, Hq + 2 Hkv, 128] -> q, k, v with the q/k RMS-norm and the rotary rotation."""

    @staticmethod
    def forward(ctx, qkv, n_q_heads, cos, sin, gamma_q, gamma_k, eps):
        qc = qkv.contiguous()
        cos = None if cos is None else cos.float().contiguous()
        sin = None if sin is None else sin.float().contiguous()
        ctx.save_for_backward(qc, cos, sin, gamma_q, gamma_k)
        ctx.eps = float(eps)
        return _k().qkv_post_fwd(qc, n_q_heads, cos, sin, gamma_q, gamma_k, eps)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, cos, sin, gq, gk = ctx.saved_tensors
        heads = qkv.shape[-2]
        rows = qkv.numel() // (heads * 128)
        # head counts come from whichever gradient exists; an output that was not used has no gradient
        hq = dq.numel() // (rows * 128) if dq is not None else None
        hk = (dk if dk is not None else dv).numel() // (rows * 128) if (dk is not None or dv is not None) else None
        if hq is None:
            hq = heads - 2 * hk
        if hk is None:
            hk = (heads - hq) // 2
        z = lambda h: torch.zeros(rows, h, 128, dtype=qkv.dtype, device=qkv.device)  # noqa: E731
        dq = z(hq) if dq is None else dq.contiguous()
        dk = z(hk) if dk is None else dk.contiguous()
        dv = z(hk) if dv is None else dv.contiguous()
        d_qkv, part = _k().qkv_post_bwd(qkv, dq, dk, dv, cos, sin, gq, gk, ctx.eps)
        sums = part.sum(0)
        dgq = sums[0].to(gq.dtype) if (gq is not None and ctx.needs_input_grad[4]) else None
        dgk = sums[1].to(gk.dtype) if (gk is not None and ctx.needs_input_grad[5]) else None
        return d_qkv, None, None, None, dgq, dgk, None


class SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        gu = gate_up.contiguous()
        ctx.save_for_backward(gu)
        return _k().swiglu(gu)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        return _k().swiglu_bwd(gu, dy.contiguous())


class GatedResidualFn(torch.autograd.Function):
    """y = x + gate[b] * f."""

    @staticmethod
    def forward(ctx, x, f, gate, rows_per_batch):
        fc = f.contiguous()
        ctx.save_for_backward(fc, gate)
        ctx.rpb = int(rows_per_batch)
        return _k().gated_residual(x.contiguous(), fc, gate, rows_per_batch)

    @staticmethod
    def backward(ctx, dy):
        f, gate = ctx.saved_tensors
        if gate is None:
            return dy, dy, None, None
        df, part = _k().gated_residual_bwd(dy.contiguous(), f, gate, ctx.rpb)
        dgate = _sum_to(part.sum(1), gate) if ctx.needs_input_grad[2] else None
        return dy, df, dgate, None


def adaln_rmsnorm(x, gamma, shift, scale, rows_per_batch: int, eps: float = 1e-6):
    return AdaLNRMSNormFn.apply(x, gamma, shift, scale, rows_per_batch, eps)


def rmsnorm(x, gamma, eps: float = 1e-6):
    return RMSNormFn.apply(x, gamma, eps)


def qkv_post(qkv, n_q_heads: int, cos, sin, gamma_q, gamma_k, eps: float = 1e-6):
    return QKVPostFn.apply(qkv, n_q_heads, cos, sin, gamma_q, gamma_k, eps)


def swiglu(gate_up):
    return SwiGLUFn.apply(gate_up)


def gated_residual(x, f, gate=None, rows_per_batch: int = 1):
    return GatedResidualFn.apply(x, f, gate, rows_per_batch)

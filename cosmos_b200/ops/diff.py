"""Differentiable CUDA definitions used while a call needs an autograd graph (training).

When gradients are required on a GPU, linear layers and attention run the autograd functions of
`autograd.py` (forward and backward GEMMs / attention on this package's tcgen05 kernels) and the
element-wise epilogues are composed from PyTorch ops. Setting COSMOS_TRAIN_LIBRARY_BACKWARD=1
switches to the library baseline (cuBLAS matmuls and fused SDPA) for A/B comparison."""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import reference as ref
from .reference import EPI_GATED_RESID, EPI_PLAIN, EPI_SWIGLU, MASK_CAUSAL, MASK_FULL, MASK_MOT


def _own_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and os.environ.get("COSMOS_TRAIN_LIBRARY_BACKWARD") != "1"


def gemm(a, w, bias=None, epi: int = EPI_PLAIN, resid=None, gate=None, rows_per_batch: int = 0):
    if _own_kernels(a) and w.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0:
        from . import autograd as own
        acc = own.linear(a, w)
        if bias is not None:
            acc = acc + bias
    else:
        acc = F.linear(a, w, bias)
    own_ew = _own_kernels(acc) and acc.shape[-1] % 16 == 0
    if epi == EPI_SWIGLU:
        if own_ew:
            from . import autograd as own
            return own.swiglu(acc)
        g, u = acc.chunk(2, dim=-1)
        return F.silu(g) * u
    if epi == EPI_GATED_RESID:
        n = acc.shape[-1]
        if own_ew and resid.dtype == torch.bfloat16:
            from . import _gate_ok
            if _gate_ok(acc, gate, rows_per_batch):
                from . import autograd as own
                return own.gated_residual(resid.reshape(acc.shape), acc, gate, rows_per_batch if gate is not None else 1)
        flat = acc.reshape(-1, n)
        if gate is not None:
            flat = flat * ref._rows_to_batch(gate, flat.shape[0], rows_per_batch)
        return (resid.reshape(-1, n) + flat).reshape(acc.shape)
    return acc


def attention(q, k, v, scale: Optional[float] = None, mask: int = MASK_FULL, n_ar: int = 0,
              return_lse: bool = False):
    if return_lse:
        return ref.attention(q, k, v, scale, mask, n_ar, True)
    if _own_kernels(q) and q.shape[-1] == 128:
        from . import autograd as own
        return own.attention(q, k, v, scale, mask, n_ar), None
    b, sq, hq, d = q.shape
    skv = k.shape[1]
    qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    m = None
    causal = False
    if mask == MASK_CAUSAL and sq == skv:
        causal = True
    elif mask != MASK_FULL:
        m = ref.attention_mask(sq, skv, mask, n_ar, q.device)
    o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=m, is_causal=causal, scale=scale,
                                       enable_gqa=(k.shape[2] != hq))
    return o.permute(0, 2, 1, 3), None

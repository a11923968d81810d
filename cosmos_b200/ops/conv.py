"""Ops of the video tokenizer: temporally-causal 3D convolution and the fused channel
RMS-norm + SiLU. CUDA bf16 channels-last-3d tensors run the implicit-GEMM kernel of
csrc/conv3d.cu when it is built; everything else runs the PyTorch definition."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch
import torch.nn.functional as F


def conv3d_causal_ref(x, weight, bias, stride: Sequence[int], spatial_pad: Tuple[int, int]):
    """x [B, C, T(+front context), H, W]: no temporal padding is added here (the caller has
    already prepended the causal context); H and W are zero-padded symmetrically."""
    return F.conv3d(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype), tuple(stride),
                    (0, spatial_pad[0], spatial_pad[1]))


def channel_rmsnorm_silu_ref(x, gamma, eps: float, silu: bool):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=1, keepdim=True) + eps) * gamma.float().view(1, -1, 1, 1, 1)
    if silu:
        y = F.silu(y)
    return y.to(x.dtype)


def _cuda_kernel_ok(x: torch.Tensor) -> bool:
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        return False
    from . import load_extension
    return load_extension() and hasattr(torch.ops.cosmos_b200, "conv3d_causal")


def conv3d_causal(x, weight, bias, stride: Sequence[int], spatial_pad: Tuple[int, int]):
    if _cuda_kernel_ok(x) and not (x.requires_grad or weight.requires_grad):
        return torch.ops.cosmos_b200.conv3d_causal(x, weight, bias, list(stride), list(spatial_pad))
    return conv3d_causal_ref(x, weight, bias, stride, spatial_pad)


def channel_rmsnorm_silu(x, gamma, eps: float = 1e-6, silu: bool = True):
    if _cuda_kernel_ok(x) and hasattr(torch.ops.cosmos_b200, "channel_rmsnorm_silu") and not x.requires_grad:
        return torch.ops.cosmos_b200.channel_rmsnorm_silu(x, gamma, eps, silu)
    return channel_rmsnorm_silu_ref(x, gamma, eps, silu)

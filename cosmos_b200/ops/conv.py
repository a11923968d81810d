"""PyTorch definitions of the video tokenizer's ops: temporally-causal 3D convolution and the channel
RMS-norm + SiLU. They run training through the tokenizer, every tokenizer whose channel widths are not multiples
of 64, and the CPU path, and they are the oracle of the channels-last encoder and decoder. The inference hot path
does not go through this module: `models/vae_cuda.py` runs encoder and decoder on the implicit-GEMM tcgen05 kernel
(`torch.ops.cosmos_b200.conv3d_cl`, `rmsnorm_silu`, `upsample_cl`, `conv_out_rgb`)."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch
import torch.nn.functional as F


def conv3d_causal(x, weight, bias, stride: Sequence[int], spatial_pad: Tuple[int, int]):
    """x [B, C, T(+front context), H, W]: no temporal padding is added here (the caller has
    already prepended the causal context); H and W are zero-padded symmetrically."""
    return F.conv3d(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype), tuple(stride),
                    (0, spatial_pad[0], spatial_pad[1]))


def channel_rmsnorm_silu(x, gamma, eps: float = 1e-6, silu: bool = True):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=1, keepdim=True) + eps) * gamma.float().view(1, -1, 1, 1, 1)
    if silu:
        y = F.silu(y)
    return y.to(x.dtype)



"""Causal 3D-convolution video tokenizer (VAE): 8x spatial, 4x temporal compression with the
first frame encoded alone, 16 latent channels. A clip of 1 + 4k frames maps to 1 + k latent
frames (the reference's `condition_frame_indexes_vision = range(19)` for 73 pixel frames,
evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb:508,682, is (73-1)/4+1 = 19).

Every convolution is causal in time (zero padding in front only) and every normalisation is a
per-position channel RMS norm, so encode/decode can run in temporal chunks with a small
per-layer cache and give exactly the same result as one pass over the whole clip.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import conv as conv_ops


class CausalConv3d(nn.Module):
    def __init__(self, cin: int, cout: int, k: Tuple[int, int, int] = (3, 3, 3),
                 stride: Tuple[int, int, int] = (1, 1, 1)):
        super().__init__()
        self.k, self.stride = k, stride
        self.weight = nn.Parameter(torch.empty(cout, cin, *k))
        self.bias = nn.Parameter(torch.zeros(cout))
        nn.init.normal_(self.weight, std=(1.0 / (cin * k[0] * k[1] * k[2])) ** 0.5)

    def forward(self, x: torch.Tensor, cache: Optional[Dict] = None) -> torch.Tensor:
        """x [B, C, T, H, W]. With `cache` (a dict shared across chunks) the temporal context comes
        from the previous chunk instead of zero padding."""
        kt, st = self.k[0], self.stride[0]
        keep = kt - st  # frames of context the next chunk needs
        key = id(self)
        if cache is not None and key in cache:
            ctx = cache[key]
        else:
            ctx = x.new_zeros(x.shape[0], x.shape[1], kt - 1, x.shape[3], x.shape[4])
        xin = torch.cat([ctx, x], dim=2) if ctx.shape[2] > 0 else x
        if cache is not None:
            cache[key] = xin[:, :, xin.shape[2] - keep:].detach() if keep > 0 else x[:, :, :0]
        return conv_ops.conv3d_causal(xin, self.weight, self.bias, self.stride,
                                      (self.k[1] // 2, self.k[2] // 2))


class ChannelRMSNorm(nn.Module):
    def __init__(self, c: int, eps: float = 1e-6):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(c))
        self.eps = eps

    def forward(self, x):
        return conv_ops.channel_rmsnorm_silu(x, self.gamma, self.eps, silu=False)


class NormSiLU(ChannelRMSNorm):
    def forward(self, x):
        return conv_ops.channel_rmsnorm_silu(x, self.gamma, self.eps, silu=True)


class ResBlock(nn.Module):
    def __init__(self, cin: int, cout: int):
        super().__init__()
        self.n1, self.c1 = NormSiLU(cin), CausalConv3d(cin, cout)
        self.n2, self.c2 = NormSiLU(cout), CausalConv3d(cout, cout)
        self.skip = CausalConv3d(cin, cout, (1, 1, 1)) if cin != cout else None

    def forward(self, x, cache=None):
        h = self.c1(self.n1(x), cache)
        h = self.c2(self.n2(h), cache)
        return h + (x if self.skip is None else self.skip(x, cache))


class Down(nn.Module):
    def __init__(self, c: int, temporal: bool):
        super().__init__()
        self.conv = CausalConv3d(c, c, (3, 3, 3), (2 if temporal else 1, 2, 2))

    def forward(self, x, cache=None):
        return self.conv(x, cache)


class Up(nn.Module):
    """Nearest-neighbour upsample (x2 in space, optionally x2 in time) followed by a conv. The
    very first output frame of a clip is not duplicated, so 1 + k frames become 1 + 2k."""

    def __init__(self, c: int, cout: int, temporal: bool):
        super().__init__()
        self.temporal = temporal
        self.conv = CausalConv3d(c, cout)

    def forward(self, x, cache=None, first_chunk: bool = True):
        if self.temporal:
            x = x.repeat_interleave(2, dim=2)
            if first_chunk:
                x = x[:, :, 1:]
        x = F.interpolate(x, scale_factor=(1, 2, 2), mode="nearest")
        return self.conv(x, cache)


class CausalVideoVAE(nn.Module):
    def __init__(self, latent_channels: int = 16, widths: Sequence[int] = (32, 64, 128, 128),
                 in_channels: int = 3):
        super().__init__()
        w = list(widths)
        self.latent_channels = latent_channels
        # encoder: 3 downsamples (all spatial, last two temporal)
        self.enc_in = CausalConv3d(in_channels, w[0])
        self.enc_blocks = nn.ModuleList()
        self.enc_down = nn.ModuleList()
        for i in range(3):
            self.enc_blocks.append(ResBlock(w[i], w[i + 1]))
            self.enc_down.append(Down(w[i + 1], temporal=(i >= 1)))
        self.enc_mid = ResBlock(w[3], w[3])
        self.enc_norm = NormSiLU(w[3])
        self.enc_out = CausalConv3d(w[3], 2 * latent_channels)
        # decoder mirrors it
        self.dec_in = CausalConv3d(latent_channels, w[3])
        self.dec_mid = ResBlock(w[3], w[3])
        self.dec_blocks = nn.ModuleList()
        self.dec_up = nn.ModuleList()
        for i in range(3):
            cin, cout = w[3 - i], w[2 - i]
            self.dec_blocks.append(ResBlock(cin, cin))
            self.dec_up.append(Up(cin, cout, temporal=(i <= 1)))
        self.dec_norm = NormSiLU(w[0])
        self.dec_out = CausalConv3d(w[0], in_channels)

    # ---- one chunk
    def _encode_chunk(self, x, cache):
        h = self.enc_in(x, cache)
        for blk, down in zip(self.enc_blocks, self.enc_down):
            h = down(blk(h, cache), cache)
        h = self.enc_mid(h, cache)
        return self.enc_out(self.enc_norm(h), cache)

    def _decode_chunk(self, z, cache, first_chunk):
        h = self.dec_mid(self.dec_in(z, cache), cache)
        for blk, up in zip(self.dec_blocks, self.dec_up):
            h = up(blk(h, cache), cache, first_chunk)
        return self.dec_out(self.dec_norm(h), cache)

    # ---- public
    def encode(self, video: torch.Tensor, chunk_frames: Optional[int] = None, sample: bool = False,
               generator=None) -> torch.Tensor:
        """video [B, 3, 1+4k, H, W] in [-1, 1] -> latent [B, C, 1+k, H/8, W/8] (the mean, unless `sample`)."""
        t = video.shape[2]
        assert (t - 1) % 4 == 0, "frame count must be 1 + 4k"
        if chunk_frames is None:
            moments = self._encode_chunk(video, None)
        else:
            assert chunk_frames % 4 == 0
            cache: Dict = {}
            outs = [self._encode_chunk(video[:, :, :1], cache)]
            for s in range(1, t, chunk_frames):
                outs.append(self._encode_chunk(video[:, :, s:s + chunk_frames], cache))
            moments = torch.cat(outs, dim=2)
        mean, logvar = moments.chunk(2, dim=1)
        if sample:
            return mean + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(
                mean.shape, generator=generator, device=mean.device, dtype=mean.dtype)
        return mean

    def decode(self, z: torch.Tensor, chunk_latents: Optional[int] = None) -> torch.Tensor:
        """latent [B, C, 1+k, h, w] -> video [B, 3, 1+4k, 8h, 8w] in roughly [-1, 1]."""
        if chunk_latents is None:
            return self._decode_chunk(z, None, True)
        cache: Dict = {}
        outs = []
        for s in range(0, z.shape[2], chunk_latents):
            outs.append(self._decode_chunk(z[:, :, s:s + chunk_latents], cache, s == 0))
        return torch.cat(outs, dim=2)

    @staticmethod
    def to_uint8(video: torch.Tensor) -> torch.Tensor:
        """[B, 3, T, H, W] in [-1, 1] -> [B, T, H, W, 3] uint8."""
        v = ((video.float().clamp(-1, 1) + 1.0) * 127.5).round().to(torch.uint8)
        return v.permute(0, 2, 3, 4, 1).contiguous()

    @staticmethod
    def from_uint8(frames: torch.Tensor) -> torch.Tensor:
        """[B, T, H, W, 3] uint8 -> [B, 3, T, H, W] in [-1, 1]."""
        return frames.permute(0, 4, 1, 2, 3).float() / 127.5 - 1.0

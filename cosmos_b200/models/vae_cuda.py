"""Tokenizer decoder on the sm_100a kernels: activations live in zero-padded channels-last volumes
[frames, H + 2, W + 2, C] (bf16), every 3x3x3 causal convolution is an implicit GEMM on the tensor
cores (each filter tap is a row-shifted TMA view of the flattened volume), the channel RMS-norm +
SiLU, the nearest upsampling and the final RGB convolution + uint8 conversion are bandwidth
kernels. Decoding runs in temporal chunks; the causal context of every convolution (the last two
frames of its input) is carried from chunk to chunk, so the result equals one pass over the clip.

Built from a `CausalVideoVAE` (same weights); requires channel widths that are multiples of 64.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .vae import CausalVideoVAE, ResBlock

TPAD = 2  # context frames in front of every volume (temporal kernel 3, stride 1)


def _pack_weight(w: torch.Tensor, cin_pad: int) -> torch.Tensor:
    """[Cout, Cin, 3, 3, 3] -> [Cout, 27 * cin_pad] bf16, tap-major (kt, kh, kw) then channel."""
    cout, cin = w.shape[:2]
    p = torch.zeros(cout, 3, 3, 3, cin_pad, dtype=torch.bfloat16, device=w.device)
    p[..., :cin] = w.permute(0, 2, 3, 4, 1).to(torch.bfloat16)
    return p.reshape(cout, 27 * cin_pad).contiguous()


class CLDecoder:
    def __init__(self, vae: CausalVideoVAE):
        dev = next(vae.parameters()).device
        assert dev.type == "cuda", "the channels-last decoder runs on CUDA"
        self.device = dev
        self.latent_channels = vae.latent_channels
        self.w: Dict[str, torch.Tensor] = {}
        self.b: Dict[str, torch.Tensor] = {}
        self.g: Dict[str, torch.Tensor] = {}

        def conv(name, m, cin_pad=None):
            cin = m.weight.shape[1]
            assert m.k == (3, 3, 3) and m.stride == (1, 1, 1)
            cp = cin_pad or cin
            assert cp % 64 == 0 and m.weight.shape[0] % 32 == 0, "channel widths must be multiples of 64"
            self.w[name] = _pack_weight(m.weight.data, cp)
            self.b[name] = m.bias.data.to(torch.bfloat16).contiguous()

        def res(name, blk: ResBlock):
            assert blk.skip is None
            self.g[name + ".n1"] = blk.n1.gamma.data.to(torch.bfloat16).contiguous()
            self.g[name + ".n2"] = blk.n2.gamma.data.to(torch.bfloat16).contiguous()
            conv(name + ".c1", blk.c1)
            conv(name + ".c2", blk.c2)

        conv("in", vae.dec_in, 64)
        res("mid", vae.dec_mid)
        self.ups: List[bool] = []
        for i, (blk, up) in enumerate(zip(vae.dec_blocks, vae.dec_up)):
            res(f"b{i}", blk)
            conv(f"u{i}", up.conv)
            self.ups.append(up.temporal)
        self.g["out"] = vae.dec_norm.gamma.data.to(torch.bfloat16).contiguous()
        wo = vae.dec_out.weight.data  # [3, 64, 3, 3, 3]
        assert wo.shape[0] == 3 and wo.shape[1] == 64, "the RGB head expects 64 input channels"
        self.w_out = wo.permute(0, 2, 3, 4, 1).reshape(3, 27, 64).float().contiguous()
        self.b_out = vae.dec_out.bias.data.float().contiguous()
        self.eps = vae.dec_norm.eps

    # ------------------------------------------------------------------ building blocks
    def _ctx(self, cache: Dict, key: str, vol: torch.Tensor) -> None:
        """Fills the context frames of `vol` from the previous chunk and remembers this chunk's tail."""
        if key in cache:
            vol[:TPAD].copy_(cache[key])
        else:
            vol[:TPAD].zero_()
        cache[key] = vol[-TPAD:].clone()

    def _conv(self, cache, name, vol, resid=None):
        self._ctx(cache, name, vol)
        out = torch.zeros(vol.shape[0], vol.shape[1], vol.shape[2], self.w[name].shape[0], dtype=torch.bfloat16,
                          device=self.device)
        torch.ops.cosmos_b200.conv3d_cl(vol, self.w[name], self.b[name], resid, out, TPAD)
        return out

    def _ns(self, vol, gamma):
        return torch.ops.cosmos_b200.rmsnorm_silu(vol, gamma, self.eps)

    def _res(self, cache, name, x):
        h = self._conv(cache, name + ".c1", self._ns(x, self.g[name + ".n1"]))
        return self._conv(cache, name + ".c2", self._ns(h, self.g[name + ".n2"]), resid=x)

    def _up(self, cache, name, x, temporal, first):
        t_src = x.shape[0] - TPAD
        t_dst = (2 * t_src - 1 if first else 2 * t_src) if temporal else t_src
        hs, ws = x.shape[1] - 2, x.shape[2] - 2
        dst = torch.zeros(t_dst + TPAD, 2 * hs + 2, 2 * ws + 2, x.shape[3], dtype=torch.bfloat16, device=self.device)
        torch.ops.cosmos_b200.upsample_cl(x, dst, TPAD, temporal, first)
        return self._conv(cache, name, dst)

    # ------------------------------------------------------------------ public
    @torch.no_grad()
    def decode_chunk(self, z: torch.Tensor, cache: Dict, first: bool) -> torch.Tensor:
        """z [C, tc, h, w] -> uint8 frames [T, 8h, 8w, 3]."""
        c, tc, h, w = z.shape
        vol = torch.zeros(tc + TPAD, h + 2, w + 2, 64, dtype=torch.bfloat16, device=self.device)
        vol[TPAD:, 1:-1, 1:-1, :c] = z.permute(1, 2, 3, 0).to(torch.bfloat16)
        x = self._conv(cache, "in", vol)
        x = self._res(cache, "mid", x)
        for i, temporal in enumerate(self.ups):
            x = self._res(cache, f"b{i}", x)
            x = self._up(cache, f"u{i}", x, temporal, first)
        x = self._ns(x, self.g["out"])
        self._ctx(cache, "out", x)
        return torch.ops.cosmos_b200.conv_out_rgb(x, self.w_out, self.b_out)

    @torch.no_grad()
    def decode(self, z: torch.Tensor, chunk_latents: int = 2) -> torch.Tensor:
        """z [1, C, T, h, w] -> uint8 [1, T_pix, 8h, 8w, 3]."""
        assert z.shape[0] == 1
        cache: Dict = {}
        outs = []
        for s in range(0, z.shape[2], chunk_latents):
            outs.append(self.decode_chunk(z[0, :, s:s + chunk_latents], cache, s == 0))
        return torch.cat(outs, dim=0)[None]


def even_frames(t0: int, n: int):
    """Temporal stride 2 over a chunk of `n` frames whose first frame has index `t0` in its level's timeline: the
    causal strided convolution keeps the frames with an even index. Returns (offset of the first kept frame inside
    the chunk, number of kept frames, index of the first kept frame in the next level's timeline)."""
    first = t0 % 2
    return first, max(0, (n - first + 1) // 2), (t0 + 1) // 2


class CLEncoder:
    """Tokenizer encoder on the same kernels as `CLDecoder`: padded channels-last volumes, every 3x3x3 causal
    convolution an implicit GEMM on the tensor cores, channel RMS-norm + SiLU as a bandwidth kernel.

    * A strided convolution (the three down-sampling steps: stride 2 in space, the last two also in time) is the
      stride-1 convolution evaluated everywhere followed by a strided copy of its even positions: causal padding
      in time and `k // 2` padding in space make output (j, i) of the strided form equal output (2j, 2i) of the
      stride-1 form. The tensor cores do 4x / 8x the minimal work on those three layers (about a third of the
      encoder's FLOPs at 720p) in exchange for one kernel for every convolution.
    * The 1x1x1 skip projections of the widening blocks are plain GEMMs over all positions of the padded volume;
      the border positions (which must stay zero, they are the next convolution's padding) are cleared afterwards.
    * The RGB input is padded to 64 channels.

    Frames are encoded in temporal chunks (the first frame alone, then `chunk_frames` at a time); each
    convolution's two context frames are carried over, so the result equals one pass over the clip.
    Reference behaviour: the tokenizer's causal encoder, cosmos_framework/inference (Wan2.2-style 4x8x8 VAE)."""

    def __init__(self, vae: CausalVideoVAE):
        dev = next(vae.parameters()).device
        assert dev.type == "cuda", "the channels-last encoder runs on CUDA"
        self.device = dev
        self.latent_channels = vae.latent_channels
        self.w: Dict[str, torch.Tensor] = {}
        self.b: Dict[str, torch.Tensor] = {}
        self.g: Dict[str, torch.Tensor] = {}
        self.eps = vae.enc_norm.eps

        def conv(name, m, cin_pad=None):
            assert m.k == (3, 3, 3)
            cp = cin_pad or m.weight.shape[1]
            assert cp % 64 == 0 and m.weight.shape[0] % 32 == 0, "channel widths must be multiples of 64"
            self.w[name] = _pack_weight(m.weight.data, cp)
            self.b[name] = m.bias.data.to(torch.bfloat16).contiguous()

        def res(name, blk: ResBlock):
            self.g[name + ".n1"] = blk.n1.gamma.data.to(torch.bfloat16).contiguous()
            self.g[name + ".n2"] = blk.n2.gamma.data.to(torch.bfloat16).contiguous()
            conv(name + ".c1", blk.c1)
            conv(name + ".c2", blk.c2)
            if blk.skip is not None:
                self.w[name + ".skip"] = blk.skip.weight.data.reshape(blk.skip.weight.shape[0], -1).to(torch.bfloat16).contiguous()
                self.b[name + ".skip"] = blk.skip.bias.data.to(torch.bfloat16).contiguous()

        conv("in", vae.enc_in, 64)
        self.downs: List[bool] = []
        for i, (blk, down) in enumerate(zip(vae.enc_blocks, vae.enc_down)):
            res(f"b{i}", blk)
            conv(f"d{i}", down.conv)
            assert down.conv.stride[1:] == (2, 2)
            self.downs.append(down.conv.stride[0] == 2)
        res("mid", vae.enc_mid)
        self.g["out"] = vae.enc_norm.gamma.data.to(torch.bfloat16).contiguous()
        conv("out", vae.enc_out)

    _ctx = CLDecoder._ctx
    _ns = CLDecoder._ns

    def _conv(self, cache, name, vol, resid=None):
        self._ctx(cache, name, vol)
        out = torch.zeros(vol.shape[0], vol.shape[1], vol.shape[2], self.w[name].shape[0], dtype=torch.bfloat16,
                          device=self.device)
        torch.ops.cosmos_b200.conv3d_cl(vol, self.w[name], self.b[name], resid, out, TPAD)
        return out

    def _res(self, cache, name, x):
        h = self._conv(cache, name + ".c1", self._ns(x, self.g[name + ".n1"]))
        if name + ".skip" in self.w:
            from .. import ops
            w = self.w[name + ".skip"]
            r = ops.gemm(x.view(-1, x.shape[-1]), w, bias=self.b[name + ".skip"]).view(*x.shape[:3], w.shape[0])
            r[:, 0].zero_(); r[:, -1].zero_(); r[:, :, 0].zero_(); r[:, :, -1].zero_()   # the padding ring stays zero
        else:
            r = x
        return self._conv(cache, name + ".c2", self._ns(h, self.g[name + ".n2"]), resid=r)

    def _down(self, cache, name, x, temporal: bool, t0: int):
        """Stride-1 convolution, then the even positions. `t0`: index of the chunk's first frame in this level's
        timeline (temporal steps keep the frames with an even index)."""
        y = self._conv(cache, name, x)
        body = y[TPAD:]
        if temporal:
            first, _, t0 = even_frames(t0, body.shape[0])
            body = body[first::2]
        hs, ws = (x.shape[1] - 2) // 2, (x.shape[2] - 2) // 2
        dst = torch.zeros(body.shape[0] + TPAD, hs + 2, ws + 2, y.shape[3], dtype=torch.bfloat16, device=self.device)
        dst[TPAD:, 1:-1, 1:-1] = body[:, 1:-1:2, 1:-1:2]
        return dst, t0

    @torch.no_grad()
    def encode_chunk(self, frames: torch.Tensor, cache: Dict, t0: int) -> torch.Tensor:
        """frames [3, n, H, W] in [-1, 1] (global index of the first one: t0) -> moments [2C, n', H/8, W/8] fp32."""
        c, n, h, w = frames.shape
        vol = torch.zeros(n + TPAD, h + 2, w + 2, 64, dtype=torch.bfloat16, device=self.device)
        vol[TPAD:, 1:-1, 1:-1, :c] = frames.permute(1, 2, 3, 0).to(torch.bfloat16)
        x = self._conv(cache, "in", vol)
        for i, temporal in enumerate(self.downs):
            x = self._res(cache, f"b{i}", x)
            x, t0 = self._down(cache, f"d{i}", x, temporal, t0)
        x = self._res(cache, "mid", x)
        y = self._conv(cache, "out", self._ns(x, self.g["out"]))
        return y[TPAD:, 1:-1, 1:-1].permute(3, 0, 1, 2).float()

    @torch.no_grad()
    def encode(self, video: torch.Tensor, chunk_frames: int = 8) -> torch.Tensor:
        """video [1, 3, 1 + 4k, H, W] in [-1, 1] (H, W multiples of 8) -> latent mean [1, C, 1 + k, H/8, W/8] fp32."""
        assert video.shape[0] == 1 and (video.shape[2] - 1) % 4 == 0 and chunk_frames % 4 == 0
        assert video.shape[3] % 8 == 0 and video.shape[4] % 8 == 0
        cache: Dict = {}
        t = video.shape[2]
        outs = [self.encode_chunk(video[0, :, :1], cache, 0)]
        for s in range(1, t, chunk_frames):
            outs.append(self.encode_chunk(video[0, :, s:s + chunk_frames], cache, s))
        moments = torch.cat(outs, dim=1)
        return moments[None, :self.latent_channels]

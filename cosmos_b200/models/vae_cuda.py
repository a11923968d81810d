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

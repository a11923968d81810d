"""Sound tokenizer: a 1-D convolutional autoencoder between stereo 48 kHz waveforms and latent
frames (reference: stereo AAC 48 kHz muxed into the MP4, README.md:109-111;
`pipe.sound_tokenizer.config.sampling_rate`, run_with_diffusers.ipynb:607)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class SoundTokenizerConfig:
    sampling_rate: int = 48000
    channels: int = 2
    latent_dim: int = 64
    hop: int = 1920  # 48000 / 1920 = 25 latent frames per second


class SoundTokenizer(nn.Module):
    def __init__(self, latent_dim: int = 64, width: int = 64, config: SoundTokenizerConfig = None):
        super().__init__()
        self.config = config or SoundTokenizerConfig(latent_dim=latent_dim)
        c = self.config
        strides = [8, 8, 6, 5]
        assert math.prod(strides) == c.hop
        enc, dec = [], []
        cin = c.channels
        for i, s in enumerate(strides):
            cout = width * min(2 ** i, 4)
            enc += [nn.Conv1d(cin, cout, 2 * s, s, s // 2), nn.SiLU()]
            cin = cout
        enc += [nn.Conv1d(cin, c.latent_dim, 3, 1, 1)]
        self.encoder = nn.Sequential(*enc)
        cin = c.latent_dim
        for i, s in enumerate(reversed(strides)):
            cout = width * min(2 ** (len(strides) - 1 - i), 4)
            dec += [nn.ConvTranspose1d(cin, cout, 2 * s, s, s // 2), nn.SiLU()]
            cin = cout
        dec += [nn.Conv1d(cin, c.channels, 7, 1, 3), nn.Tanh()]
        self.decoder = nn.Sequential(*dec)

    def latent_frames(self, seconds: float) -> int:
        return max(1, int(round(seconds * self.config.sampling_rate / self.config.hop)))

    def encode(self, wav: torch.Tensor) -> torch.Tensor:
        """wav [B, N, 2] in [-1, 1] -> latents [B, T, latent_dim]."""
        return self.encoder(wav.transpose(1, 2)).transpose(1, 2)

    def decode(self, lat: torch.Tensor) -> torch.Tensor:
        """latents [B, T, latent_dim] -> wav [B, T*hop, 2]."""
        w = self.decoder(lat.transpose(1, 2)).transpose(1, 2)
        return w[:, :lat.shape[1] * self.config.hop]

"""Stand-ins for the three media helpers the reference's Diffusers notebook imports from `diffusers.utils`
(`load_image`, `export_to_video`, `encode_video`; reference
cookbooks/cosmos3/generator/audiovisual/run_with_diffusers.ipynb, the cell that defines `run_payload`), on top of
this package's own readers and writers, with the call shapes used there."""
from __future__ import annotations

from pathlib import Path
from typing import Optional, Sequence, Union

import numpy as np

from ..io import media


def _as_frames(video) -> np.ndarray:
    """uint8 [T, H, W, 3] from an array (uint8, or float in [0, 1]) or a sequence of arrays / PIL images."""
    if isinstance(video, np.ndarray):
        arr = video
    else:
        arr = np.stack([np.asarray(f) for f in video])
    if arr.dtype != np.uint8:
        arr = (np.clip(arr.astype(np.float32), 0.0, 1.0) * 255.0).round().astype(np.uint8)
    if arr.ndim == 3:
        arr = arr[None]
    return arr


def load_image(path_or_image):
    """A PIL RGB image from a path (or an image, passed through)."""
    from PIL import Image

    if isinstance(path_or_image, Image.Image):
        return path_or_image.convert("RGB")
    if str(path_or_image).startswith(("http://", "https://")):
        raise ValueError("remote images are not fetched; download the file and pass its path")
    return Image.open(path_or_image).convert("RGB")


def export_to_video(video, output_video_path: Union[str, Path], fps: int = 24, quality: int = 8,
                    macro_block_size: Optional[int] = None) -> str:
    """Writes frames to an MP4 and returns the path. `macro_block_size` is accepted and ignored (no resizing is
    ever applied here)."""
    media.write_video(Path(output_video_path), _as_frames(video), fps, quality, None, 48000)
    return str(output_video_path)


def encode_video(video, fps: int, output_path: Union[str, Path], audio: Optional[Sequence] = None,
                 audio_sample_rate: int = 48000, quality: int = 8) -> str:
    """Frames plus an optional sound track ([N, 2] or [2, N] float in [-1, 1]) into one MP4."""
    snd = None
    if audio is not None:
        snd = np.asarray(audio.detach().cpu().float().numpy() if hasattr(audio, "detach") else audio, dtype=np.float32)
        if snd.ndim == 2 and snd.shape[0] <= 2 < snd.shape[1]:
            snd = snd.T
    media.write_video(Path(output_path), _as_frames(video), fps, quality, snd, audio_sample_rate)
    return str(output_path)

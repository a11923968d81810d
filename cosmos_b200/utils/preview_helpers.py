"""Helpers for looking at video-transfer runs: load one of the control specs, resolve the paths
inside it, and make a small preview clip of a result (same role as the reference's notebook helper
cookbooks/cosmos3/generator/transfer/preview_helpers.py, which shells out to ffmpeg libx264 crf 28;
here a preview is re-encoded with ffmpeg when it is installed and with the built-in Motion-JPEG
writer at half resolution otherwise)."""
from __future__ import annotations

import json
import os
import subprocess
from pathlib import Path
from typing import Optional

import numpy as np

from ..io import media

CONTROLS = ("edge", "blur", "depth", "seg", "wsm")


def specs_dir() -> Path:
    """Directory with `<control>.json` specs: $COSMOS3_TRANSFER_SPECS or ./specs."""
    return Path(os.environ.get("COSMOS3_TRANSFER_SPECS", "specs"))


def output_root() -> Path:
    return Path(os.environ.get("COSMOS3_OUTPUT_ROOT", "outputs")) / "transfer"


def resolve_spec_path(path_str: str, base: Optional[Path] = None) -> Path:
    """Paths inside a spec are relative to the spec file's directory."""
    p = Path(path_str)
    return p if p.is_absolute() else ((base or specs_dir()) / p).resolve()


def load_transfer_spec(control: str, directory: Optional[Path] = None) -> dict:
    if control not in CONTROLS:
        raise ValueError(f"control must be one of {CONTROLS}")
    path = (directory or specs_dir()) / f"{control}.json"
    spec = json.loads(path.read_text())
    if control not in spec:
        raise ValueError(f"{path} has no '{control}' hint block")
    return spec


def make_preview(src: Path, crf: int = 28, max_frames: Optional[int] = None) -> Path:
    """Writes `<src stem>_preview.mp4` next to `src` and returns its path."""
    src = Path(src)
    dst = src.with_name(src.stem + "_preview.mp4")
    if media.have_ffmpeg():
        cmd = ["ffmpeg", "-y", "-v", "error", "-i", str(src), "-c:v", "libx264", "-crf", str(crf), "-pix_fmt",
               "yuv420p", "-an", str(dst)]
        if subprocess.run(cmd).returncode == 0:
            return dst
    frames, fps = media.read_video(src, max_frames)
    small = np.ascontiguousarray(frames[:, ::2, ::2])
    media.write_video(dst, small, fps, quality=4, prefer_ffmpeg=False)
    return dst


def preview_transfer(control: str, directory: Optional[Path] = None) -> dict:
    """Previews of the control video and of the generated result (when it exists)."""
    spec = load_transfer_spec(control, directory)
    base = directory or specs_dir()
    out = {"control": None, "result": None}
    ctrl = resolve_spec_path(spec[control]["control_path"], base)
    if ctrl.exists():
        out["control"] = make_preview(ctrl)
    result = output_root() / spec["name"] / "vision.mp4"
    if result.exists():
        out["result"] = make_preview(result)
    return out

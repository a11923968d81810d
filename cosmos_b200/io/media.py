"""Media I/O: images via PIL, videos via an `ffmpeg` binary when one is on PATH and via the
built-in Motion-JPEG MP4 muxer otherwise. Outputs follow the reference layout
(`<out>/<name>/vision.mp4`, images as PNG; stereo 48 kHz audio muxed into the MP4,
reference README.md:109-111)."""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path
from typing import Optional, Tuple

import numpy as np

from . import mp4


def have_ffmpeg() -> bool:
    return shutil.which("ffmpeg") is not None


def read_image(path, size: Optional[Tuple[int, int]] = None) -> np.ndarray:
    """-> [H, W, 3] uint8; `size` = (width, height) resizes with centre crop to the aspect ratio."""
    from PIL import Image

    img = Image.open(path).convert("RGB")
    if size is not None:
        img = _resize_center_crop(img, size)
    return np.asarray(img)


def _resize_center_crop(img, size):
    from PIL import Image

    w, h = size
    sw, sh = img.size
    scale = max(w / sw, h / sh)
    nw, nh = max(w, round(sw * scale)), max(h, round(sh * scale))
    img = img.resize((nw, nh), Image.BICUBIC)
    left, top = (nw - w) // 2, (nh - h) // 2
    return img.crop((left, top, left + w, top + h))


def write_image(path, frame: np.ndarray) -> None:
    from PIL import Image

    Image.fromarray(np.ascontiguousarray(frame)).save(path)


def read_video(path, max_frames: Optional[int] = None, size: Optional[Tuple[int, int]] = None, start: int = 0
               ) -> Tuple[np.ndarray, float]:
    """-> (frames [T, H, W, 3] uint8, fps), at most `max_frames` frames from frame `start` on. Supports .npy/.npz
    frame arrays, image files (1 frame), this package's Motion-JPEG MP4 natively, other codecs (H.264, HEVC,
    AV1, ...) through OpenCV's bundled decoders (which seek to `start`), else through an ffmpeg binary."""
    from PIL import Image

    path = Path(path)
    suffix = path.suffix.lower()
    if suffix == ".npy":
        frames, fps = np.load(path), 24.0
    elif suffix == ".npz":
        z = np.load(path)
        frames, fps = z["frames"], float(z["fps"]) if "fps" in z else 24.0
    elif suffix in (".png", ".jpg", ".jpeg", ".bmp", ".webp"):
        frames, fps = read_image(path)[None], 1.0
    else:
        want = None if max_frames is None else start + max_frames
        try:
            frames, fps = mp4.read_mp4_mjpeg(path, want)
        except ValueError:
            # not one of this package's own Motion-JPEG files: OpenCV's bundled decoders (H.264, HEVC, AV1, ...)
            # when OpenCV is installed, else the ffmpeg binary
            got = _opencv_read(path, max_frames, start)
            if got is not None:
                start = 0                      # already skipped by seeking
            else:
                if not have_ffmpeg():
                    raise
                got = _ffmpeg_read(path, want)
            frames, fps = got
    if start:
        frames = frames[start:]
    if max_frames is not None:
        frames = frames[:max_frames]
    if size is not None and (frames.shape[2], frames.shape[1]) != tuple(size):
        frames = np.stack([np.asarray(_resize_center_crop(Image.fromarray(f), size)) for f in frames])
    return frames, fps


def sample_video(path, fps: Optional[float] = None, num_frames: Optional[int] = None, limit: int = 32
                 ) -> Tuple[np.ndarray, list, float]:
    """Frames of a clip sampled in time -> (frames [n, H, W, 3] uint8, their times in seconds, source fps).
    `num_frames` > 0 spreads that many frames evenly over the clip; else `fps` keeps every round(src_fps / fps)-th
    frame; with neither every frame is kept. At most `limit` frames come back. With OpenCV the frames in between
    are skipped in the decoder and never converted or stored, so a long clip costs the memory of its samples."""
    path = Path(path)
    cap = None
    if path.suffix.lower() not in (".npy", ".npz", ".png", ".jpg", ".jpeg", ".bmp", ".webp"):
        try:
            import cv2
            cap = cv2.VideoCapture(str(path))
            if not cap.isOpened():
                cap = None
        except ImportError:
            cap = None
    if cap is None:
        frames, src_fps = read_video(path)
        idx = _sample_indices(len(frames), src_fps, fps, num_frames, limit)
        return frames[idx], (idx / max(src_fps, 1e-6)).tolist(), src_fps
    try:
        import cv2
        src_fps = float(cap.get(cv2.CAP_PROP_FPS)) or 24.0
        total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        if total <= 0:                       # container without a frame count: decode everything once
            cap.release()
            frames, src_fps = read_video(path)
            idx = _sample_indices(len(frames), src_fps, fps, num_frames, limit)
            return frames[idx], (idx / max(src_fps, 1e-6)).tolist(), src_fps
        idx = _sample_indices(total, src_fps, fps, num_frames, limit)
        want, out, kept, pos = set(idx.tolist()), [], [], 0
        last = int(idx[-1]) if len(idx) else -1
        while pos <= last:
            if not cap.grab():
                break
            if pos in want:
                ok, bgr = cap.retrieve()
                if ok:
                    out.append(bgr[:, :, ::-1])
                    kept.append(pos)
            pos += 1
    finally:
        cap.release()
    if not out:
        raise ValueError(f"no frame could be decoded from {path}")
    return np.ascontiguousarray(np.stack(out)), [k / max(src_fps, 1e-6) for k in kept], src_fps


def _sample_indices(n: int, src_fps: float, fps: Optional[float], num_frames: Optional[int], limit: int) -> np.ndarray:
    idx = np.arange(n)
    if num_frames and num_frames > 0:
        idx = np.linspace(0, max(n - 1, 0), int(num_frames)).round().astype(np.int64)
    elif fps:
        idx = idx[::max(1, int(round(src_fps / max(float(fps), 1e-6))))]
    return idx[:limit]


def _opencv_read(path, max_frames, start: int = 0) -> Optional[Tuple[np.ndarray, float]]:
    """Decodes a video with OpenCV's FFmpeg backend -> (frames RGB uint8, fps); None when OpenCV is missing or
    cannot open the file."""
    try:
        import cv2
    except ImportError:
        return None
    cap = cv2.VideoCapture(str(path))
    try:
        if not cap.isOpened():
            return None
        fps = float(cap.get(cv2.CAP_PROP_FPS)) or 24.0
        if start:
            cap.set(cv2.CAP_PROP_POS_FRAMES, int(start))
            if int(cap.get(cv2.CAP_PROP_POS_FRAMES)) != int(start):   # container without an index: decode and drop
                cap.set(cv2.CAP_PROP_POS_FRAMES, 0)
                for _ in range(int(start)):
                    if not cap.grab():
                        break
        frames = []
        while max_frames is None or len(frames) < max_frames:
            ok, bgr = cap.read()
            if not ok:
                break
            frames.append(bgr[:, :, ::-1])
    finally:
        cap.release()
    if not frames:
        return None
    return np.ascontiguousarray(np.stack(frames)), fps


def _ffmpeg_read(path, max_frames):
    probe = subprocess.run(["ffprobe", "-v", "error", "-select_streams", "v:0", "-show_entries",
                            "stream=width,height,r_frame_rate", "-of", "csv=p=0", str(path)],
                           capture_output=True, text=True, check=True).stdout.strip().split(",")
    w, h = int(probe[0]), int(probe[1])
    num, den = probe[2].split("/")
    cmd = ["ffmpeg", "-v", "error", "-i", str(path)]
    if max_frames:
        cmd += ["-frames:v", str(max_frames)]
    cmd += ["-f", "rawvideo", "-pix_fmt", "rgb24", "-"]
    raw = subprocess.run(cmd, capture_output=True, check=True).stdout
    return np.frombuffer(raw, np.uint8).reshape(-1, h, w, 3), float(num) / float(den)


def write_video(path, frames: np.ndarray, fps: float, quality: int = 8, audio: Optional[np.ndarray] = None,
                sample_rate: int = 48000, prefer_ffmpeg: bool = True) -> str:
    """Writes `frames` [T, H, W, 3] uint8 as MP4; returns the codec used ('h264' or 'mjpeg')."""
    frames = np.ascontiguousarray(frames)
    if prefer_ffmpeg and have_ffmpeg() and audio is None:
        t, h, w, _ = frames.shape
        crf = int(np.clip(36 - 2 * quality, 10, 40))
        cmd = ["ffmpeg", "-y", "-v", "error", "-f", "rawvideo", "-pix_fmt", "rgb24", "-s", f"{w}x{h}", "-r",
               str(fps), "-i", "-", "-c:v", "libx264", "-pix_fmt", "yuv420p", "-crf", str(crf), str(path)]
        r = subprocess.run(cmd, input=frames.tobytes(), capture_output=True)
        if r.returncode == 0:
            return "h264"
    mp4.write_mp4_mjpeg(path, frames, fps, quality, audio, sample_rate)
    return "mjpeg"

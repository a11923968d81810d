"""Self-contained MP4 (ISO BMFF) writer/reader for Motion-JPEG video with optional 16-bit PCM
stereo audio. It exists so that the framework can emit the reference's `vision.mp4` output
(reference cookbooks/cosmos3/generator/action/run_fd_with_cosmos_framework.ipynb:629) on a box
with no ffmpeg, PyAV or torchcodec; when an `ffmpeg` binary is on PATH, `media.write_video`
prefers H.264 through it. Files written here are read back by `read_mp4_mjpeg` (used by the
autoregressive chunk loops that feed the last frame of one chunk into the next) and are
playable by ffmpeg/VLC/QuickTime, which all support the `jpeg` sample entry.
"""
from __future__ import annotations

import io
import struct
from typing import List, Optional, Tuple

import numpy as np


def _box(kind: bytes, payload: bytes) -> bytes:
    return struct.pack(">I4s", 8 + len(payload), kind) + payload


def _full(kind: bytes, version: int, flags: int, payload: bytes) -> bytes:
    return _box(kind, struct.pack(">B3s", version, flags.to_bytes(3, "big")) + payload)


_MATRIX = struct.pack(">9I", 0x10000, 0, 0, 0, 0x10000, 0, 0, 0, 0x40000000)


def _trak(track_id: int, handler: bytes, name: bytes, timescale: int, duration: int, movie_duration: int,
          stsd_entry: bytes, media_header: bytes, sample_sizes: List[int], sample_delta: int,
          chunk_offsets: List[int], samples_per_chunk: int, width: int = 0, height: int = 0,
          volume: int = 0) -> bytes:
    tkhd = _full(b"tkhd", 0, 7, struct.pack(">IIIII", 0, 0, track_id, 0, movie_duration) + bytes(8)
                 + struct.pack(">hhhH", 0, 0, volume, 0) + _MATRIX + struct.pack(">II", width << 16, height << 16))
    mdhd = _full(b"mdhd", 0, 0, struct.pack(">IIIIHH", 0, 0, timescale, duration, 0x55C4, 0))
    hdlr = _full(b"hdlr", 0, 0, struct.pack(">I4s", 0, handler) + bytes(12) + name + b"\0")
    dinf = _box(b"dinf", _full(b"dref", 0, 0, struct.pack(">I", 1) + _full(b"url ", 0, 1, b"")))
    stsd = _full(b"stsd", 0, 0, struct.pack(">I", 1) + stsd_entry)
    n = len(sample_sizes)
    stts = _full(b"stts", 0, 0, struct.pack(">III", 1, n, sample_delta))
    stsc = _full(b"stsc", 0, 0, struct.pack(">IIII", 1, 1, samples_per_chunk, 1))
    if len(set(sample_sizes)) == 1 and n > 0 and samples_per_chunk != 1:
        stsz = _full(b"stsz", 0, 0, struct.pack(">II", sample_sizes[0], n))
    else:
        stsz = _full(b"stsz", 0, 0, struct.pack(">II", 0, n) + b"".join(struct.pack(">I", s) for s in sample_sizes))
    co64 = _full(b"co64", 0, 0, struct.pack(">I", len(chunk_offsets))
                 + b"".join(struct.pack(">Q", o) for o in chunk_offsets))
    stbl = _box(b"stbl", stsd + stts + stsc + stsz + co64)
    minf = _box(b"minf", media_header + dinf + stbl)
    mdia = _box(b"mdia", mdhd + hdlr + minf)
    return _box(b"trak", tkhd + mdia)


def encode_jpeg_frames(frames: np.ndarray, quality: int = 8) -> List[bytes]:
    """frames [T, H, W, 3] uint8; `quality` is the CLI's 0..10 scale (--video-save-quality)."""
    from PIL import Image

    q = int(np.clip(35 + 6 * quality, 1, 95))
    out = []
    for f in frames:
        buf = io.BytesIO()
        Image.fromarray(np.ascontiguousarray(f)).save(buf, format="JPEG", quality=q)
        out.append(buf.getvalue())
    return out


def write_mp4_mjpeg(path, frames: np.ndarray, fps: float, quality: int = 8,
                    audio: Optional[np.ndarray] = None, sample_rate: int = 48000) -> None:
    """frames [T, H, W, 3] uint8; audio (optional) float [-1, 1] or int16, shape [N, 2] (stereo)."""
    frames = np.asarray(frames)
    assert frames.ndim == 4 and frames.shape[-1] == 3 and frames.dtype == np.uint8
    t, h, w, _ = frames.shape
    jpegs = encode_jpeg_frames(frames, quality)
    timescale = 30000
    delta = int(round(timescale / float(fps)))
    vdur = delta * t
    pcm = b""
    n_audio = 0
    if audio is not None:
        a = np.asarray(audio)
        if a.ndim == 1:
            a = np.stack([a, a], axis=-1)
        if a.dtype != np.int16:
            a = (np.clip(a.astype(np.float64), -1, 1) * 32767.0).round().astype(np.int16)
        n_audio = a.shape[0]
        pcm = a.astype(">i2").tobytes()  # 'twos' = big-endian signed PCM
    ftyp = _box(b"ftyp", b"isom" + struct.pack(">I", 0x200) + b"isomiso2mp41qt  ")
    mdat_payload_off = len(ftyp) + 16  # 64-bit mdat header
    offsets, off = [], mdat_payload_off
    for j in jpegs:
        offsets.append(off)
        off += len(j)
    audio_off = off
    mdat = struct.pack(">I4sQ", 1, b"mdat", 16 + sum(map(len, jpegs)) + len(pcm))
    movie_ts = 1000
    movie_dur = int(round(max(t / float(fps), n_audio / float(sample_rate) if n_audio else 0) * movie_ts))
    jpeg_entry = _box(b"jpeg", bytes(6) + struct.pack(">H", 1) + bytes(16) + struct.pack(">HHIIIH", w, h, 0x480000,
                      0x480000, 0, 1) + bytes(32) + struct.pack(">Hh", 24, -1))
    vmhd = _full(b"vmhd", 0, 1, bytes(8))
    traks = _trak(1, b"vide", b"VideoHandler", timescale, vdur, movie_dur, jpeg_entry, vmhd,
                  [len(j) for j in jpegs], delta, offsets, 1, w, h)
    if n_audio:
        twos = _box(b"twos", bytes(6) + struct.pack(">H", 1) + struct.pack(">HHIHHHHI", 0, 0, 0, 2, 16, 0, 0,
                    sample_rate << 16))
        smhd = _full(b"smhd", 0, 0, bytes(4))
        traks += _trak(2, b"soun", b"SoundHandler", sample_rate, n_audio,
                       movie_dur, twos, smhd, [4] * n_audio, 1, [audio_off], n_audio, volume=0x0100)
    mvhd = _full(b"mvhd", 0, 0, struct.pack(">IIII", 0, 0, movie_ts, movie_dur) + struct.pack(">IH", 0x10000, 0x0100)
                 + bytes(10) + _MATRIX + bytes(24) + struct.pack(">I", 3))
    moov = _box(b"moov", mvhd + traks)
    with open(path, "wb") as f:
        f.write(ftyp)
        f.write(mdat)
        for j in jpegs:
            f.write(j)
        f.write(pcm)
        f.write(moov)


# ----------------------------------------------------------------------------- reader
def _iter_boxes(buf: bytes, start: int, end: int):
    pos = start
    while pos + 8 <= end:
        size, kind = struct.unpack_from(">I4s", buf, pos)
        hdr = 8
        if size == 1:
            size = struct.unpack_from(">Q", buf, pos + 8)[0]
            hdr = 16
        elif size == 0:
            size = end - pos
        yield kind, pos + hdr, pos + size
        pos += size


def _find(buf, start, end, path):
    for kind, s, e in _iter_boxes(buf, start, end):
        if kind == path[0]:
            return (s, e) if len(path) == 1 else _find(buf, s, e, path[1:])
    return None


def read_mp4_mjpeg(path, max_frames: Optional[int] = None) -> Tuple[np.ndarray, float]:
    """Reads a file written by `write_mp4_mjpeg`; returns (frames [T, H, W, 3] uint8, fps)."""
    from PIL import Image

    buf = open(path, "rb").read()
    moov = _find(buf, 0, len(buf), [b"moov"])
    if moov is None:
        raise ValueError(f"{path}: no moov box")
    for kind, s, e in _iter_boxes(buf, *moov):
        if kind != b"trak":
            continue
        hd = _find(buf, s, e, [b"mdia", b"hdlr"])
        if hd is None or buf[hd[0] + 8:hd[0] + 12] != b"vide":
            continue
        mdhd = _find(buf, s, e, [b"mdia", b"mdhd"])
        timescale = struct.unpack_from(">I", buf, mdhd[0] + 12)[0]
        stbl = _find(buf, s, e, [b"mdia", b"minf", b"stbl"])
        stsd = _find(buf, *stbl, [b"stsd"])
        codec = buf[stsd[0] + 12:stsd[0] + 16]
        if codec not in (b"jpeg", b"mjpa", b"mjpg"):
            raise ValueError(f"{path}: video codec {codec!r} needs an external decoder (ffmpeg); "
                             "only Motion-JPEG is decoded natively")
        stts = _find(buf, *stbl, [b"stts"])
        delta = struct.unpack_from(">I", buf, stts[0] + 12)[0]
        stsz = _find(buf, *stbl, [b"stsz"])
        fixed, n = struct.unpack_from(">II", buf, stsz[0] + 4)
        sizes = [fixed] * n if fixed else list(struct.unpack_from(f">{n}I", buf, stsz[0] + 12))
        co = _find(buf, *stbl, [b"co64"])
        if co is not None:
            cnt = struct.unpack_from(">I", buf, co[0] + 4)[0]
            offs = list(struct.unpack_from(f">{cnt}Q", buf, co[0] + 8))
        else:
            co = _find(buf, *stbl, [b"stco"])
            cnt = struct.unpack_from(">I", buf, co[0] + 4)[0]
            offs = list(struct.unpack_from(f">{cnt}I", buf, co[0] + 8))
        n = min(n, len(offs)) if max_frames is None else min(n, len(offs), max_frames)
        frames = [np.asarray(Image.open(io.BytesIO(buf[offs[i]:offs[i] + sizes[i]])).convert("RGB"))
                  for i in range(n)]
        return np.stack(frames), timescale / float(delta)
    raise ValueError(f"{path}: no video track")

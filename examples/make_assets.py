"""Writes the small synthetic media the example specs point at (a conditioning image, a short
conditioning / control video, an action chunk) into examples/assets/, so that every example runs
without any download:

    python examples/make_assets.py
"""
import json
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from cosmos_b200.io import media  # noqa: E402


def scene(t: int, h: int = 192, w: int = 320) -> np.ndarray:
    """A smooth moving gradient with a bright square (compresses well, has motion and edges)."""
    y, x = np.mgrid[0:h, 0:w].astype(np.float32)
    img = np.stack([(x / w * 200 + 3 * t) % 255, y / h * 220, (x + y) / (h + w) * 255], -1)
    x0 = 20 + 6 * t
    img[60:110, x0:x0 + 50] = (250, 240, 90)
    return img.astype(np.uint8)


def main(out: Path = Path(__file__).resolve().parent / "assets") -> None:
    out.mkdir(parents=True, exist_ok=True)
    media.write_image(out / "first_frame.png", scene(0))
    frames = np.stack([scene(t) for t in range(17)])
    media.write_video(out / "clip.mp4", frames, 16, 8, None, 48000)
    gray = frames.mean(-1)
    edges = (np.abs(np.diff(gray, axis=2, prepend=gray[:, :, :1])) > 8).astype(np.uint8) * 255
    media.write_video(out / "control_edge.mp4", np.repeat(edges[..., None], 3, -1), 16, 8, None, 48000)
    # 16 steps of a slow forward motion: translation (3) + rot6d (6) + gripper (1)
    act = np.tile(np.array([0.0, 0.0, 0.02, 1, 0, 0, 0, 1, 0, 0.5], dtype=np.float32), (16, 1))
    (out / "actions_droid.json").write_text(json.dumps(act.tolist()))
    print(f"assets written to {out}")


if __name__ == "__main__":
    main()

"""Guardrails: prompt screening and face blur (reference README.md:394 and
cookbooks/cosmos3/README.md:96-133: enabled by default, `--no-guardrails` turns them off; the
reference's implementation uses a text screen and RetinaFace via OpenCV, whose weights are not
available offline). The text screen here is a normalised blocklist match; the video pass blurs
the boxes returned by a pluggable face detector (none is bundled, so without one the frames pass
through unchanged and that is reported in `last_report`)."""
from __future__ import annotations

import re
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

DEFAULT_BLOCKLIST = (
    "child sexual", "csam", "bestiality", "build a bomb", "make a bomb", "synthesize nerve agent",
)


class GuardrailViolation(ValueError):
    pass


Box = Tuple[int, int, int, int]


class Guardrails:
    def __init__(self, blocklist: Sequence[str] = DEFAULT_BLOCKLIST,
                 face_detector: Optional[Callable[[np.ndarray], List[Box]]] = None, blur_kernel: int = 31):
        self.blocklist = tuple(b.lower() for b in blocklist)
        self.face_detector = face_detector
        self.blur_kernel = blur_kernel | 1
        self.last_report = {}

    @staticmethod
    def _norm(text: str) -> str:
        return re.sub(r"[^a-z0-9 ]+", " ", text.lower())

    def check_prompt(self, text: str) -> None:
        t = self._norm(text)
        for b in self.blocklist:
            if b in t:
                self.last_report = {"blocked": True, "term": b}
                raise GuardrailViolation("prompt rejected by the text guardrail")
        self.last_report = {"blocked": False}

    def blur_faces(self, frames: np.ndarray) -> np.ndarray:
        """frames [T, H, W, 3] uint8 -> same, with detected face boxes box-blurred."""
        if self.face_detector is None:
            self.last_report["face_blur"] = "no detector configured; frames unchanged"
            return frames
        out = frames.copy()
        n = 0
        for i, f in enumerate(frames):
            for (x0, y0, x1, y1) in self.face_detector(f):
                x0, y0 = max(0, x0), max(0, y0)
                x1, y1 = min(f.shape[1], x1), min(f.shape[0], y1)
                if x1 > x0 and y1 > y0:
                    out[i, y0:y1, x0:x1] = _box_blur(f[y0:y1, x0:x1], self.blur_kernel)
                    n += 1
        self.last_report["face_blur"] = f"{n} boxes blurred"
        return out


def _box_blur(img: np.ndarray, k: int) -> np.ndarray:
    pad = k // 2
    p = np.pad(img.astype(np.float32), ((pad, pad), (pad, pad), (0, 0)), mode="edge")
    c = np.cumsum(np.cumsum(p, axis=0), axis=1)
    c = np.pad(c, ((1, 0), (1, 0), (0, 0)))
    h, w = img.shape[:2]
    s = c[k:k + h, k:k + w] - c[:h, k:k + w] - c[k:k + h, :w] + c[:h, :w]
    return (s / (k * k)).round().astype(np.uint8)

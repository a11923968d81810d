"""Guardrails: prompt screening and face blur (reference README.md:394 and
cookbooks/cosmos3/README.md:96-133: enabled by default, `--no-guardrails` turns them off; the
reference's implementation uses a text screen and RetinaFace via OpenCV, whose weights are not
available offline). The text screen here is a normalised blocklist match; the video pass blurs
the boxes returned by a face detector: by default OpenCV's bundled frontal-face cascade when OpenCV is
installed (`opencv_face_detector`), a YuNet model when `COSMOS_FACE_MODEL` points at its ONNX file, or any
callable; without a detector the frames pass through unchanged and `last_report` says so."""
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


def opencv_face_detector(model_path: Optional[str] = None, min_size: int = 24) -> Optional[Callable[[np.ndarray], List[Box]]]:
    """A detector `frame [H, W, 3] uint8 RGB -> [(x0, y0, x1, y1), ...]` built on OpenCV, or None when OpenCV (or
    its cascade file) is not installed. With `model_path` (a YuNet ONNX file) `cv2.FaceDetectorYN` is used,
    otherwise the frontal-face Haar cascade that ships inside the OpenCV package."""
    try:
        import cv2
    except ImportError:
        return None
    if model_path:
        det = cv2.FaceDetectorYN.create(model_path, "", (320, 320))

        def run_yunet(frame: np.ndarray) -> List[Box]:
            h, w = frame.shape[:2]
            det.setInputSize((w, h))
            _, faces = det.detect(np.ascontiguousarray(frame[:, :, ::-1]))
            return [] if faces is None else [(int(f[0]), int(f[1]), int(f[0] + f[2]), int(f[1] + f[3])) for f in faces]

        return run_yunet
    import os
    xml = os.path.join(getattr(cv2.data, "haarcascades", ""), "haarcascade_frontalface_default.xml")
    if not os.path.exists(xml):
        return None
    cascade = cv2.CascadeClassifier(xml)
    if cascade.empty():
        return None

    def run_cascade(frame: np.ndarray) -> List[Box]:
        gray = cv2.cvtColor(np.ascontiguousarray(frame), cv2.COLOR_RGB2GRAY)
        # detection runs on a copy whose longer side is at most 480 pixels; boxes are scaled back
        scale = max(1.0, max(gray.shape) / 480.0)
        if scale > 1.0:
            gray = cv2.resize(gray, (int(round(gray.shape[1] / scale)), int(round(gray.shape[0] / scale))),
                              interpolation=cv2.INTER_AREA)
        found = cascade.detectMultiScale(gray, scaleFactor=1.1, minNeighbors=5, minSize=(min_size, min_size))
        return [(int(x * scale), int(y * scale), int(np.ceil((x + w) * scale)), int(np.ceil((y + h) * scale)))
                for (x, y, w, h) in found]

    return run_cascade


class Guardrails:
    def __init__(self, blocklist: Sequence[str] = DEFAULT_BLOCKLIST, face_detector="auto", blur_kernel: int = 31):
        """`face_detector`: "auto" (OpenCV when installed, see `opencv_face_detector`), None, or a callable
        `frame -> boxes`."""
        import os
        self.blocklist = tuple(b.lower() for b in blocklist)
        if isinstance(face_detector, str):
            if face_detector != "auto":
                raise ValueError("face_detector must be 'auto', None or a callable")
            face_detector = opencv_face_detector(os.environ.get("COSMOS_FACE_MODEL"))
        self.face_detector: Optional[Callable[[np.ndarray], List[Box]]] = face_detector
        self.blur_kernel = blur_kernel | 1
        self.last_report = {}

    @staticmethod
    def _norm(text: str) -> str:
        return re.sub(r"\s+", " ", re.sub(r"[^a-z0-9]+", " ", text.lower())).strip()

    def check_prompt(self, text: str) -> None:
        t = self._norm(text)
        for b in self.blocklist:
            if b in t:
                self.last_report = {"blocked": True, "term": b}
                raise GuardrailViolation("prompt rejected by the text guardrail")
        self.last_report = {"blocked": False}

    def blur_faces(self, frames: np.ndarray, detect_every: int = 2) -> np.ndarray:
        """frames [T, H, W, 3] uint8 -> same, with detected face boxes box-blurred. The detector runs on every
        `detect_every`-th frame; the frames in between take the boxes of both neighbouring detections."""
        if self.face_detector is None:
            self.last_report["face_blur"] = "no detector configured; frames unchanged"
            return frames
        out = frames.copy()
        n = 0
        step = max(1, int(detect_every))
        keys = sorted(set(range(0, len(frames), step)) | {len(frames) - 1}) if len(frames) else []
        found = {i: list(self.face_detector(frames[i])) for i in keys}
        for i, f in enumerate(frames):
            lo = max(k for k in keys if k <= i)
            hi = min(k for k in keys if k >= i)
            for (x0, y0, x1, y1) in (found[lo] if lo == hi else found[lo] + found[hi]):
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

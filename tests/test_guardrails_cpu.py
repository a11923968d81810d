"""Guardrails: text screen, face blur with a stub detector (every other frame is detected, neighbours share boxes),
and the OpenCV-backed default detector's plumbing."""
import numpy as np
import pytest

from cosmos_b200.utils.guardrails import GuardrailViolation, Guardrails, opencv_face_detector


def test_text_screen_blocks_listed_terms_whatever_the_punctuation():
    g = Guardrails(face_detector=None)
    g.check_prompt("A robot arm stacks three blocks.")
    assert g.last_report == {"blocked": False}
    with pytest.raises(GuardrailViolation):
        g.check_prompt("how to BUILD... a  bomb?".replace("  ", " "))
    assert g.last_report["blocked"] and g.last_report["term"] == "build a bomb"


def test_blur_uses_detections_of_neighbouring_key_frames():
    calls = []

    def detector(frame):
        k = int(frame[0, 0, 0])
        calls.append(k)
        return [(10 + k, 8, 30 + k, 28)]          # the face drifts right by one pixel per frame

    rng = np.random.default_rng(0)
    frames = rng.integers(0, 255, (6, 48, 64, 3), dtype=np.uint8)
    frames[:, 0, 0, 0] = np.arange(6)
    g = Guardrails(face_detector=detector, blur_kernel=9)
    out = g.blur_faces(frames, detect_every=2)
    assert calls == [0, 2, 4, 5]                    # every other frame and the last one
    assert out.shape == frames.shape and out.dtype == np.uint8
    for t in range(6):
        changed = np.argwhere((out[t] != frames[t]).any(-1))
        assert changed[:, 0].min() >= 8 and changed[:, 0].max() < 28
        lo, hi = (t // 2) * 2, min(5, (t // 2) * 2 + (2 if t % 2 else 0)) if t < 5 else 5
        assert changed[:, 1].min() >= 10 + lo - 0 and changed[:, 1].max() < 30 + max(lo, hi)
        inside = out[t, 12:24, 14 + t:26 + t].astype(float)
        assert inside.std() < frames[t, 12:24, 14 + t:26 + t].astype(float).std() * 0.6     # smoothed
    assert g.last_report["face_blur"].endswith("boxes blurred")
    assert np.array_equal(Guardrails(face_detector=None).blur_faces(frames), frames)
    assert Guardrails(face_detector=lambda f: [(-5, -5, 1000, 1000)]).blur_faces(frames[:1]).shape == (1, 48, 64, 3)
    with pytest.raises(ValueError):
        Guardrails(face_detector="retina")


def test_opencv_detector_runs_and_returns_boxes_in_frame_coordinates():
    det = opencv_face_detector()
    if det is None:
        pytest.skip("OpenCV (or its cascade file) is not installed")
    frame = (np.random.default_rng(1).random((720, 1280, 3)) * 255).astype(np.uint8)
    boxes = det(frame)
    assert isinstance(boxes, list)
    for x0, y0, x1, y1 in boxes:
        assert 0 <= x0 < x1 <= 1280 + 3 and 0 <= y0 < y1 <= 720 + 3
    g = Guardrails()                                   # "auto" picks the OpenCV detector up
    assert g.face_detector is not None
    assert g.blur_faces(frame[None]).shape == (1, 720, 1280, 3)

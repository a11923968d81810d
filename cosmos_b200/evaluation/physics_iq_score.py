"""Built-in scorer for the Physics-IQ evaluation: how closely the motion in a generated clip follows the real
continuation of the same scene.

The reference scores with the benchmark's own program (`run_physics_iq.py --generated_videos_dir ... --results_dir
... --physics_iq_dir ... --fps 24`, reference evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb, last
code cell), which lives in another repository and needs the benchmark download. This module restates the four
published measures (Motamed et al., "Do generative video models understand physical principles?", 2025) so that a
run can be scored where only the staged clips and the real clips are at hand; it takes the same flag names.
Scores from here track the official ones in ordering, not in the last digit: motion masks are computed here from
frame differences with a fixed threshold, not read from the benchmark's mask files.

Per clip pair (generated, real), both [T, H, W, 3] uint8 at the same size and length:
* motion map m_t = |gray_t - gray_{t-1}| and binary mask b_t = dilate3x3(m_t > threshold);
* spatial IoU ("where"):            IoU( OR_t b_t(gen), OR_t b_t(real) );
* spatiotemporal IoU ("where+when"): mean_t IoU( b_t(gen), b_t(real) ), frames without motion in both count as 1;
* weighted spatial IoU ("where+how much"): sum min(a_g, a_r) / sum max(a_g, a_r) with a = sum_t b_t (per-pixel
  amount of action);
* MSE ("how"): mean squared error of the pixels in [0, 1].
With a second real take (`--real_take2_dir`) every measure is normalised by what two real takes of the scene reach
(the physical variance) and the Physics-IQ score of a clip is the mean of the four normalised measures, capped at
100; without it the raw measures are reported and the score is their plain mean (MSE entering as 1 - min(1, MSE / 0.05)).
"""
from __future__ import annotations

import argparse
import csv
import json
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

from ..io import media

MOTION_THRESHOLD = 10.0 / 255.0
MSE_SCALE = 0.05
MEASURES = ("spatial_iou", "spatiotemporal_iou", "weighted_spatial_iou", "mse")


def motion_masks(frames: torch.Tensor, threshold: float = MOTION_THRESHOLD) -> torch.Tensor:
    """frames [T, H, W, 3] uint8 -> bool [T-1, H, W]: pixels whose brightness changed between consecutive frames,
    grown by one pixel (3x3 dilation) so that thin edges of the same motion overlap."""
    gray = frames.float().mean(-1) / 255.0
    diff = (gray[1:] - gray[:-1]).abs()
    mask = (diff > threshold).float()[:, None]
    return F.max_pool2d(mask, 3, 1, 1)[:, 0] > 0


def _iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """IoU over the last two axes; 1 where both are empty."""
    inter = (a & b).flatten(-2).sum(-1).float()
    union = (a | b).flatten(-2).sum(-1).float()
    return torch.where(union > 0, inter / union.clamp_min(1), torch.ones_like(union))


def compare(gen: np.ndarray, real: np.ndarray, device: str = "cpu") -> Dict[str, float]:
    """The four raw measures for one pair of clips."""
    if gen.shape != real.shape:
        raise ValueError(f"clips differ in shape: {gen.shape} vs {real.shape}")
    if gen.shape[0] < 2:
        raise ValueError("a clip needs at least two frames")
    g, r = torch.from_numpy(gen).to(device), torch.from_numpy(real).to(device)
    bg, br = motion_masks(g), motion_masks(r)
    ag, ar = bg.float().sum(0), br.float().sum(0)
    denom = torch.maximum(ag, ar).sum()
    weighted = (torch.minimum(ag, ar).sum() / denom).item() if denom > 0 else 1.0
    return {"spatial_iou": _iou(bg.any(0), br.any(0)).item(),
            "spatiotemporal_iou": _iou(bg, br).mean().item(),
            "weighted_spatial_iou": weighted,
            "mse": ((g.float() - r.float()) / 255.0).pow(2).mean().item()}


def physics_iq(raw: Dict[str, float], variance: Optional[Dict[str, float]] = None) -> float:
    """Score of one clip in [0, 100]. `variance` = the measures of real take 2 against real take 1."""
    if variance is None:
        parts = [raw["spatial_iou"], raw["spatiotemporal_iou"], raw["weighted_spatial_iou"],
                 1.0 - min(1.0, raw["mse"] / MSE_SCALE)]
    else:
        parts = [min(1.0, raw[k] / max(variance[k], 1e-6)) for k in MEASURES[:3]]
        parts.append(min(1.0, max(variance["mse"], 1e-6) / max(raw["mse"], 1e-6)))   # lower is better
    return 100.0 * float(np.mean(parts))


def _load(path: Path, like: Optional[np.ndarray] = None, n_frames: Optional[int] = None) -> np.ndarray:
    size = None if like is None else (like.shape[2], like.shape[1])
    frames, _ = media.read_video(path, max_frames=n_frames, size=size)
    return frames


def _find(directory: Path, case: str) -> Optional[Path]:
    for suffix in (".mp4", ".npy", ".npz"):
        p = directory / f"{case}{suffix}"
        if p.exists():
            return p
    return None


def score_directory(generated_dir, real_dir, results_dir, real_take2_dir=None, device: str = "cpu") -> Dict[str, float]:
    """Scores every clip of `generated_dir` that has a real clip of the same name (staged clips are named by case
    id); writes `<results>/per_case.csv` and `<results>/summary.json`; returns the summary."""
    generated_dir, real_dir, results_dir = Path(generated_dir), Path(real_dir), Path(results_dir)
    results_dir.mkdir(parents=True, exist_ok=True)
    rows: List[Dict[str, float]] = []
    for g_path in sorted(p for p in generated_dir.iterdir() if p.suffix.lower() in (".mp4", ".npy", ".npz")):
        case = g_path.stem
        r_path = _find(real_dir, case)
        if r_path is None:
            continue
        gen = _load(g_path)
        real = _load(r_path, like=gen, n_frames=gen.shape[0])
        n = min(gen.shape[0], real.shape[0])
        raw = compare(gen[:n], real[:n], device)
        var = None
        if real_take2_dir is not None:
            t2 = _find(Path(real_take2_dir), case)
            if t2 is not None:
                var = compare(_load(t2, like=gen, n_frames=n)[:n], real[:n], device)
        rows.append({"case": case, **raw, "physics_iq": physics_iq(raw, var)})
    if not rows:
        raise ValueError(f"no clip in {generated_dir} has a real counterpart in {real_dir}")
    with open(results_dir / "per_case.csv", "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=["case", *MEASURES, "physics_iq"])
        w.writeheader()
        w.writerows(rows)
    summary = {k: float(np.mean([r[k] for r in rows])) for k in (*MEASURES, "physics_iq")}
    summary["cases"] = len(rows)
    (results_dir / "summary.json").write_text(json.dumps(summary, indent=1))
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--generated_videos_dir", required=True, help="staged clips named <case id>.mp4 / .npy")
    ap.add_argument("--results_dir", required=True)
    ap.add_argument("--physics_iq_dir", required=True, help="folder with the real continuations, named like the staged clips")
    ap.add_argument("--real_take2_dir", default=None, help="second real take of every scene (physical variance)")
    ap.add_argument("--fps", type=int, default=24, help="accepted for compatibility; clips are compared frame by frame")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    summary = score_directory(args.generated_videos_dir, args.physics_iq_dir, args.results_dir, args.real_take2_dir,
                              args.device)
    print(json.dumps(summary))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

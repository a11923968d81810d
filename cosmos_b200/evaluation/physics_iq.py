"""PhysicsIQ reproduction harness: builds the per-case inference specs for the image-to-video and
video-to-video settings, runs them through the inference CLI and prepares the clips for the
official scorer.

Recipes (reference evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb:460-523 and
README.md:24-29): I2V = 121 frames, 50 steps, guidance 3.0 on interval [0, 1000], shift 4.75,
sigma_max 80, negative_metadata_mode "none"; V2V = 193 frames with the first 19 latent frames
(73 pixel frames) given as clean conditioning, 50 steps, guidance 6.0, shift 5.0, sigma_max 80,
negative_metadata_mode "same", negative_prompt_keep_metadata true, normalize_cfg false.
Prompt files hold 198 rows of {name, prompt, negative_prompt}. The scorer compares the 5 s after
the conditioning part at 24 fps = 120 frames, so I2V output drops its first frame (121 -> 120)
and V2V output drops the 73 conditioning frames (193 -> 120). The DeepMind scorer itself and the
PhysicsIQ videos are external downloads and are not bundled.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np

I2V_RECIPE = dict(model_mode="image2video", num_steps=50, guidance=3.0, guidance_interval=[0, 1000], shift=4.75,
                  sigma_max=80.0, num_frames=121, fps=24, resolution="720", aspect_ratio="16,9",
                  negative_metadata_mode="none", num_outputs=1, seed=0)
V2V_RECIPE = dict(model_mode="video2video", num_steps=50, guidance=6.0, shift=5.0, sigma_max=80.0, num_frames=193,
                  fps=24, resolution="720", aspect_ratio="16,9", condition_frame_indexes_vision=list(range(19)),
                  negative_metadata_mode="same", negative_prompt_keep_metadata=True, normalize_cfg=False,
                  num_outputs=1, seed=0)
N_CASES = 198
SCORED_FRAMES = 120
V2V_CONDITIONING_FRAMES = 73


def load_prompts(path) -> List[Dict[str, str]]:
    rows = json.loads(Path(path).read_text())
    for r in rows:
        if not {"name", "prompt", "negative_prompt"} <= set(r):
            raise ValueError(f"{path}: each row needs name, prompt and negative_prompt")
    return rows


def build_specs(setting: str, prompts: List[Dict[str, str]], media_dir, limit: Optional[int] = None,
                overrides: Optional[dict] = None) -> List[dict]:
    """One spec per case. `media_dir` holds the conditioning media named `<case name>.jpg` (I2V: the
    switch frame) or `<case name>.mp4` (V2V: the 3 s conditioning clip)."""
    if setting not in ("i2v", "v2v"):
        raise ValueError("setting must be 'i2v' or 'v2v'")
    recipe = dict(I2V_RECIPE if setting == "i2v" else V2V_RECIPE)
    recipe.update(overrides or {})
    ext = ".jpg" if setting == "i2v" else ".mp4"
    specs = []
    for row in prompts[:limit]:
        specs.append({**recipe, "name": row["name"], "prompt": row["prompt"], "negative_prompt": row["negative_prompt"],
                      "vision_path": str(Path(media_dir) / (row["name"] + ext))})
    return specs


def write_jsonl(specs: List[dict], path) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text("".join(json.dumps(s) + "\n" for s in specs))
    return path


def scored_frames(frames: np.ndarray, setting: str) -> np.ndarray:
    """The part of a generated clip that the scorer compares with the real continuation."""
    drop = 1 if setting == "i2v" else V2V_CONDITIONING_FRAMES
    out = frames[drop:drop + SCORED_FRAMES]
    if out.shape[0] != SCORED_FRAMES:
        raise ValueError(f"expected at least {drop + SCORED_FRAMES} frames, got {frames.shape[0]}")
    return out


def inference_command(spec_file, out_dir, checkpoint: str = "Cosmos3-Super", gpus: int = 4, cp_size: Optional[int] = None
                      ) -> List[str]:
    """`--cp-size` = all visible GPUs, as in the reference notebook (its cell with `--cp-size=$COSMOS3_NUM_GPUS`)."""
    cp = cp_size or gpus
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr",
            "127.0.0.1", "-m", "cosmos_b200.scripts.inference", "-i", str(spec_file), "-o", str(out_dir),
            "--checkpoint-path", checkpoint, "--dp-shard-size=1", "--dp-replicate-size=1", f"--cp-size={cp}",
            "--cfgp-size=1", "--no-guardrails", "--benchmark"]


def postprocess(out_dir, setting: str, names: List[str]) -> Dict[str, str]:
    """Writes `<out>/<name>/scored.npy` (120 frames) for every finished case."""
    from ..io import media

    done = {}
    for n in names:
        mp4 = Path(out_dir) / n / "vision.mp4"
        if not mp4.exists():
            continue
        frames, _ = media.read_video(mp4)
        np.save(mp4.with_name("scored.npy"), scored_frames(frames, setting))
        done[n] = str(mp4.with_name("scored.npy"))
    return done


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--setting", choices=["i2v", "v2v"], required=True)
    ap.add_argument("--prompts", required=True, help="i2v_prompts.json / v2v_prompts.json")
    ap.add_argument("--media-dir", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--checkpoint-path", default="Cosmos3-Super")
    ap.add_argument("--gpus", type=int, default=4)
    ap.add_argument("--limit", type=int, default=None)
    ap.add_argument("--dry-run", action="store_true", help="write the spec file and print the command only")
    args = ap.parse_args(argv)
    prompts = load_prompts(args.prompts)
    specs = build_specs(args.setting, prompts, args.media_dir, args.limit)
    spec_file = write_jsonl(specs, Path(args.out) / f"physics_iq_{args.setting}.jsonl")
    cmd = inference_command(spec_file, Path(args.out) / args.setting, args.checkpoint_path, args.gpus)
    print(" ".join(cmd))
    if args.dry_run:
        return 0
    rc = subprocess.run(cmd).returncode
    if rc == 0:
        postprocess(Path(args.out) / args.setting, args.setting, [s["name"] for s in specs])
    return rc


if __name__ == "__main__":
    raise SystemExit(main())

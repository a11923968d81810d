"""Every example spec under examples/ parses, and each model mode runs end to end on the tiny
model on CPU (shrunk to a few frames and one sampling step) through the same functions the CLI uses."""
import dataclasses
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from cosmos_b200.io.spec import load_specs

EX = Path(__file__).resolve().parents[1] / "examples"
FILES = sorted(p.name for p in EX.glob("*.json")) + sorted(p.name for p in EX.glob("*.jsonl"))


def test_examples_cover_every_generator_mode_and_the_reasoner():
    modes = {s.model_mode for f in FILES for s in load_specs(EX / f)}
    assert {"text2image", "text2video", "image2video", "video2video", "forward_dynamics", "inverse_dynamics",
            "reasoner"} <= modes
    for f in ("first_frame.png", "clip.mp4", "control_edge.mp4", "actions_droid.json"):
        assert (EX / "assets" / f).exists(), f"run examples/make_assets.py ({f} is missing)"


@pytest.fixture(scope="module")
def pipe():
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    torch.manual_seed(0)
    return Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=32, n_layers=1))


@pytest.mark.parametrize("fname", [f for f in FILES if f.endswith(".json")])
def test_example_runs_on_the_tiny_model(fname, pipe, tmp_path):
    from cosmos_b200.scripts import inference as cli

    spec = load_specs(EX / fname)[0]
    small = dict(num_steps=1, guidance=1.0)
    if spec.model_mode == "reasoner":
        small = dict(max_new_tokens=3)
    elif spec.model_mode in ("forward_dynamics", "inverse_dynamics"):
        small.update(image_size=256)
    else:
        small.update(resolution="256", num_frames=1 if spec.num_frames == 1 else 5)
        if spec.num_video_frames_per_chunk:
            small.update(num_video_frames_per_chunk=5)
    spec = dataclasses.replace(spec, **small)
    out = tmp_path / spec.name
    if spec.model_mode == "reasoner":
        from cosmos_b200.models.reasoner import ReasonerEngine
        from cosmos_b200.models.vit import VisionEncoder
        vit = VisionEncoder(pipe.cfg).eval()
        rec = cli.run_reasoner_sample(ReasonerEngine(pipe.transformer, vit), pipe.tokenizer, vit, spec, out, True,
                                      pipe.device)
        assert (out / "reasoner_text.txt").exists() and rec["completion_tokens"] <= 3
        return
    rec = cli.run_generator_sample(pipe, spec, out, 8, True)
    assert rec["model_mode"] == spec.model_mode and rec["generation_time_s"] > 0
    meta = json.loads((out / "sample_outputs.json").read_text())
    if spec.num_frames == 1:
        assert (out / "vision.png").exists()
    else:
        assert (out / "vision.mp4").stat().st_size > 1000
    if spec.model_mode == "inverse_dynamics":
        act = np.asarray(meta["outputs"][0]["content"]["action"])
        assert act.shape == (spec.action_chunk_size, 10) and np.isfinite(act).all()


def test_single_image_output_follows_the_diffusers_convention(pipe, tmp_path):
    """`pipe(..., num_frames=1).video[0].save(path)` as in the reference's Diffusers notebook; "np" gives the array."""
    kw = dict(prompt="a cube", num_frames=1, height=32, width=32, num_inference_steps=1, guidance_scale=1.0,
              generator=torch.Generator().manual_seed(3))
    out = pipe(**kw)
    out.video[0].save(tmp_path / "img.png")
    assert (tmp_path / "img.png").stat().st_size > 100 and out.video[0].size == (32, 32)
    arr = pipe(output_type="np", **{**kw, "generator": torch.Generator().manual_seed(3)}).video
    assert arr.shape == (1, 32, 32, 3) and np.array_equal(np.asarray(out.video[0]), arr[0])
    with pytest.raises(ValueError):
        pipe(output_type="pt", **kw)


def test_generation_is_deterministic_by_seed(pipe):
    """Same spec and seed -> identical frames; another seed -> different frames."""
    import torch
    kw = dict(prompt="a ball rolls", num_frames=5, height=32, width=32, fps=8, num_inference_steps=2, guidance_scale=3.0)
    a = pipe(generator=torch.Generator().manual_seed(7), **kw).video
    b = pipe(generator=torch.Generator().manual_seed(7), **kw).video
    c = pipe(generator=torch.Generator().manual_seed(8), **kw).video
    assert np.array_equal(np.asarray(a), np.asarray(b))
    assert not np.array_equal(np.asarray(a), np.asarray(c))


def test_forward_dynamics_rollout_chains_chunks_on_the_last_frame(pipe):
    """12 actions in chunks of 4 -> three chunks, 13 frames; chunk k starts from chunk k - 1's last frame."""
    rng = np.random.default_rng(0)
    acts = rng.normal(0, 0.05, (12, 9)).astype(np.float32)
    start = (rng.random((32, 32, 3)) * 255).astype(np.uint8)
    seen = []
    out = pipe.forward_dynamics_rollout(start, acts, action_chunk_size=4, domain=0, height=32, width=32, fps=10, seed=5,
                                        num_inference_steps=1, guidance_scale=1.0, callback=lambda k, n: seen.append((k, n)))
    assert out.video.shape == (13, 32, 32, 3) and seen == [(0, 3), (1, 3), (2, 3)]
    # the second chunk on its own, started from frame 4 of the rollout with seed 5 + 1, reproduces frames 4..8
    again = pipe(prompt="", image=out.video[4], num_frames=5, height=32, width=32, fps=10, action=acts[4:8], domain=0,
                 action_dim=9, num_inference_steps=1, guidance_scale=1.0, output_type="np",
                 generator=torch.Generator().manual_seed(6))
    assert np.array_equal(again.video[1:], out.video[5:9])
    with pytest.raises(ValueError):
        pipe.forward_dynamics_rollout(start, acts[:10], action_chunk_size=4, height=32, width=32)


def test_video_transfer_control_stream_steers_the_generation(pipe):
    """The control clip runs as a second clean vision stream in a third guidance branch: another control clip or
    another `control_guidance` changes the result, weight 0 reproduces the generation without a control clip, and
    chunked generation hands every chunk its own stretch of the control clip."""
    from cosmos_b200.config import SamplingConfig
    rng = np.random.default_rng(3)
    ctrl_a = (rng.random((5, 32, 32, 3)) * 255).astype(np.uint8)
    ctrl_b = (rng.random((5, 32, 32, 3)) * 255).astype(np.uint8)
    kw = dict(prompt="a robot arm", num_frames=5, height=32, width=32, fps=8, output_type="latent")

    def run(control, cg, weight=1.0):
        sc = SamplingConfig(num_steps=2, guidance=3.0, shift=3.0, scheduler="euler", seed=11, control_guidance=cg)
        extra = {} if control is None else {"control_video": control, "control_weight": weight}
        return pipe(sampling=sc, **kw, **extra).latents

    base = run(None, None)
    a15 = run(ctrl_a, 1.5)
    assert not torch.allclose(a15, base)
    assert not torch.allclose(run(ctrl_b, 1.5), a15)            # the control clip matters
    assert not torch.allclose(run(ctrl_a, 0.5), a15)            # and so does its guidance scale
    assert torch.allclose(run(ctrl_a, 0.0), base, atol=1e-6)    # scale 0 = no control
    assert torch.allclose(run(ctrl_a, 1.5, weight=0.0), base, atol=1e-6)
    # chunked: 9 frames in chunks of 5 with 1 conditioning frame -> chunk 1 sees control frames 4..8
    seen = []
    orig = pipe.prepare

    def spy(*a, **k):
        seen.append(None if k.get("control_video") is None else np.asarray(k["control_video"]).copy())
        return orig(*a, **k)

    long_ctrl = (rng.random((9, 32, 32, 3)) * 255).astype(np.uint8)
    pipe.prepare = spy
    try:
        sc = SamplingConfig(num_steps=1, guidance=2.0, shift=3.0, scheduler="euler", seed=1, control_guidance=1.0)
        out = pipe.generate_chunked("a robot arm", num_frames=9, height=32, width=32, fps=8, frames_per_chunk=5,
                                    num_conditional_frames=1, sampling=sc, control_video=long_ctrl, output_type="np")
    finally:
        pipe.prepare = orig
    assert out.video.shape[0] == 9 and len(seen) == 2
    assert np.array_equal(seen[0], long_ctrl[0:5]) and np.array_equal(seen[1], long_ctrl[4:9])

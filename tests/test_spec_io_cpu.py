"""Spec parser/validator, pose utilities, MP4 muxer, tokenizer: CPU-only contract tests."""
import json
import os
from pathlib import Path

import numpy as np
import pytest

from cosmos_b200.data.vfm.action import pose_utils
from cosmos_b200.io import media, mp4
from cosmos_b200.io.spec import SpecError, load_specs, spec_from_dict
from cosmos_b200.utils.tokenizer import ByteTokenizer

# the reference checkout, when it sits next to this repository (its cookbook specs serve as parsing fixtures)
REF = Path(os.environ.get("COSMOS_REFERENCE_DIR", Path(__file__).resolve().parents[2] / "reference"))


def test_t2v_defaults_match_recipe():
    s = spec_from_dict({"model_mode": "text2video", "name": "a", "prompt": "x"})
    assert (s.num_steps, s.guidance, s.shift, s.num_frames, s.fps, s.resolution) == (35, 6.0, 10.0, 189, 24, "720")
    assert not s.is_transfer and s.is_generator


def test_json_vs_jsonl_and_relative_paths(tmp_path):
    (tmp_path / "p.json").write_text(json.dumps({"subjects": [], "fps": 24}))
    one = {"model_mode": "text2video", "name": "a", "prompt_path": "p.json"}
    (tmp_path / "one.json").write_text(json.dumps(one))
    (tmp_path / "many.jsonl").write_text(json.dumps(one) + "\n\n" + json.dumps({**one, "name": "b"}) + "\n")
    a = load_specs(tmp_path / "one.json")
    assert len(a) == 1 and a[0].resolve(a[0].prompt_path) == tmp_path / "p.json"
    assert a[0].prompt_text() == '{"subjects":[],"fps":24}'  # compact JSON string
    b = load_specs(tmp_path / "many.jsonl")
    assert [s.name for s in b] == ["a", "b"]
    (tmp_path / "dup.jsonl").write_text(json.dumps(one) + "\n" + json.dumps(one) + "\n")
    with pytest.raises(SpecError):
        load_specs(tmp_path / "dup.jsonl")


@pytest.mark.parametrize("bad", [
    {"model_mode": "text2video", "name": "a", "bogus_key": 1},
    {"model_mode": "nope", "name": "a"},
    {"model_mode": "reasoner", "name": "a", "enable_sound": True},
    {"model_mode": "text2video", "name": "a", "num_frames": 120},
    {"model_mode": "text2video", "name": "a", "resolution": "1080"},
    {"model_mode": "text2video", "name": "a", "fps": 25},
    {"model_mode": "text2video", "name": "a", "vision_path": "x.jpg"},
    {"model_mode": "image2video", "name": "a"},
    {"model_mode": "text2image", "name": "a", "num_frames": 5},
    {"model_mode": "text2video", "name": "a", "control_guidance": 1.5},
    {"model_mode": "text2video", "name": "a", "edge": {"control_path": "c.mp4"}},
    {"model_mode": "video2video", "name": "a", "vision_path": "v.mp4", "edge": {"control_path": "c.mp4"},
     "num_outputs": 2},
    {"model_mode": "forward_dynamics", "name": "a", "vision_path": "i.jpg", "domain_name": "av"},
    {"model_mode": "forward_dynamics", "name": "a", "vision_path": "i.jpg", "domain_name": "mars",
     "action_chunk_size": 60, "action_path": "a.json"},
    {"model_mode": "text2video", "name": "a", "guidance": "high"},
    {"model_mode": "text2video", "name": "a/b"},
    {"model_mode": "video2video", "name": "a", "vision_path": "v.mp4", "num_frames": 193,
     "condition_frame_indexes_vision": [49]},
])
def test_strict_rejection(bad):
    with pytest.raises(SpecError):
        spec_from_dict(bad)


def test_action_modes_and_overrides():
    s = spec_from_dict({"model_mode": "forward_dynamics", "name": "fd", "vision_path": "i.jpg", "domain_name": "av",
                        "action_chunk_size": 60, "action_path": "a.json", "image_size": 480, "view_point": "ego_view"})
    assert s.num_frames == 61 and s.guidance == 1.0 and s.fps == 10 and s.resolution == "480"
    s2 = spec_from_dict({"model_mode": "inverse_dynamics", "name": "id", "vision_path": "v.mp4",
                         "domain_name": "av", "action_chunk_size": 60, "raw_action_dim": 9},
                        overrides={"image_size": 256, "seed": 7})
    assert s2.image_size == 256 and s2.seed == 7 and s2.resolution == "256"


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
def test_reference_transfer_specs_parse():
    specs_dir = REF / "cookbooks/cosmos3/generator/transfer/specs"
    for name in ("edge", "blur", "depth", "seg", "wsm"):
        (s,) = load_specs(specs_dir / f"{name}.json")
        assert s.is_transfer and name in s.controls and s.model_mode == "video2video"
        assert s.num_steps == 50 and s.share_vision_temporal_positions is True
        assert s.control_guidance in (1.5, 2.0, 3.0)
    (w,) = load_specs(specs_dir / "wsm.json")
    assert (w.num_frames, w.fps, w.guidance) == (101, 10, 1.0)


def test_rot6d_roundtrip_and_orthonormal():
    rng = np.random.default_rng(0)
    q, _ = np.linalg.qr(rng.normal(size=(5, 3, 3)))
    q[np.linalg.det(q) < 0, :, 2] *= -1
    d6 = pose_utils.rotmat_to_rot6d(q)
    r = pose_utils.rot6d_to_rotmat(d6)
    assert np.allclose(r, q, atol=1e-9)
    assert np.allclose(r @ np.swapaxes(r, -1, -2), np.eye(3), atol=1e-9)


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
@pytest.mark.parametrize("traj", ["forward", "left", "right"])
def test_pose_roundtrip_on_reference_trajectories(traj):
    path = REF / f"cookbooks/cosmos3/generator/action/assets/actions/av_traj_{traj}.json"
    act = np.asarray(json.loads(path.read_text()), dtype=np.float64)
    assert act.shape == (60, 9)
    poses = pose_utils.pose_rel_to_abs(act, "rot6d", "backward_framewise", 1.35)
    assert poses.shape == (61, 4, 4) and np.allclose(poses[0], np.eye(4))
    back = pose_utils.pose_abs_to_rel(poses, "rot6d", "backward_framewise", 1.35)
    # the stored rot6d need not be exactly orthonormal; compare through the rotation it encodes
    assert np.allclose(back[:, :3], act[:, :3], atol=1e-8)
    assert np.allclose(pose_utils.rot6d_to_rotmat(back[:, 3:]), pose_utils.rot6d_to_rotmat(act[:, 3:]), atol=1e-8)


def test_mp4_roundtrip_with_audio(tmp_path):
    yy, xx = np.mgrid[0:48, 0:64]
    base = np.stack([xx * 2, yy * 3, (xx + yy)], axis=-1).astype(np.uint8)[None]
    frames = np.repeat(base, 5, axis=0)
    frames[:, :, :, 0] = (np.arange(5)[:, None, None] * 40).astype(np.uint8)
    audio = np.sin(np.linspace(0, 100, 9600))[:, None].repeat(2, 1)
    p = tmp_path / "vision.mp4"
    mp4.write_mp4_mjpeg(p, frames, 24, 10, audio, 48000)
    got, fps = mp4.read_mp4_mjpeg(p)
    assert got.shape == frames.shape and abs(fps - 24) < 0.01
    assert np.abs(got[..., 0].astype(int).mean(axis=(1, 2)) - frames[..., 0].mean(axis=(1, 2))).max() < 6
    data = p.read_bytes()
    assert data[4:8] == b"ftyp" and b"moov" in data and b"jpeg" in data and b"twos" in data
    codec = media.write_video(tmp_path / "v2.mp4", frames, 24)
    f2, _ = media.read_video(tmp_path / "v2.mp4") if codec == "mjpeg" else (frames, 24)
    assert f2.shape == frames.shape


def test_byte_tokenizer_roundtrip_and_chat():
    tok = ByteTokenizer(32000)
    text = "héllo <think>x</think>"
    ids = tok.encode(text)
    assert tok.decode(ids, skip_special=False) == text
    assert len(tok.pad_or_truncate(ids, 512)) == 512
    chat = tok.apply_chat_template([{"role": "user", "content": [
        {"type": "image_url", "image_url": {"url": "x"}}, {"type": "text", "text": "what?"}]}], True, [4])
    assert chat.count(tok.image_pad_id) == 4
    assert tok.decode(chat, skip_special=False).endswith("<|im_start|>assistant\n")


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
def test_droid_lerobot_dataset_items():
    from cosmos_b200.data.vfm.action.datasets import DROIDLeRobotDataset

    root = REF / "cookbooks/cosmos3/generator/action/assets/droid_lerobot_example"
    ds = DROIDLeRobotDataset(root, action_chunk_size=16, decode_video=False)
    assert ds.fps == 15 and len(ds) == (722 - 16 + 15) // 16
    item = ds[0]
    assert item["action"].shape == (16, 10) and item["action"].dtype == np.float32
    assert item["conditioning_fps"] == 15 and isinstance(item["ai_caption"], str)
    r = pose_utils.rot6d_to_rotmat(item["action"][:, 3:9].astype(np.float64))
    assert np.allclose(r @ np.swapaxes(r, -1, -2), np.eye(3), atol=1e-5)
    assert np.abs(item["action"][:, :3]).max() < 0.2  # metres moved per frame at 15 fps


def test_policy_runner_returns_action_chunk():
    import torch
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    from cosmos_b200.scripts.action_policy_server_robolab import PolicyRunner

    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=16, n_layers=1))
    runner = PolicyRunner(pipe)
    img = (np.random.rand(48, 64, 3) * 255).astype(np.uint8)
    out = runner.act({"instruction": "pick up the cube", "image": img.tolist(), "domain_name": "droid_lerobot",
                      "action_chunk_size": 4, "image_size": 64, "num_steps": 2})
    assert out["shape"] == [4, 10] and np.isfinite(np.asarray(out["action"])).all()


def test_chunked_long_video_generation():
    """Chunk plan arithmetic, and a 13-frame clip generated as chunks of 9 frames with one
    conditioning frame carried from chunk to chunk."""
    import torch
    from cosmos_b200.pipeline import Cosmos3OmniPipeline, _chunk_plan

    assert _chunk_plan(121, 121, 0, 1, 4) == [(0, 121, 121)]
    assert _chunk_plan(241, 121, 0, 1, 4) == [(0, 121, 121), (1, 120, 121)]
    assert _chunk_plan(13, 9, 0, 1, 4) == [(0, 9, 9), (1, 4, 5)]
    assert _chunk_plan(20, 9, 5, 1, 4) == [(5, 4, 9), (1, 8, 9), (1, 8, 9)]
    with pytest.raises(ValueError):
        _chunk_plan(20, 1, 0, 1, 4)
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=16, n_layers=1))
    seen = []
    orig = pipe.prepare

    def spy(*a, **kw):
        seen.append((a[4] if len(a) > 4 else kw.get("num_frames"), kw.get("condition_frame_indexes")))
        return orig(*a, **kw)

    pipe.prepare = spy
    out = pipe.generate_chunked("a ball rolls", num_frames=13, height=32, width=32, fps=8, frames_per_chunk=9,
                                num_conditional_frames=1, num_inference_steps=2, guidance_scale=1.0)
    assert np.asarray(out.video).shape == (13, 32, 32, 3) and out.timings["chunks"] == 2
    assert seen == [(9, None), (5, [0])]


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
def test_physics_iq_specs_validate(tmp_path):
    from cosmos_b200.evaluation import physics_iq as piq

    for setting in ("i2v", "v2v"):
        prompts = piq.load_prompts(REF / f"evaluation/cosmos3/Physics_IQ/assets/{setting}_prompts.json")
        assert len(prompts) == piq.N_CASES
        specs = piq.build_specs(setting, prompts, tmp_path, limit=3)
        f = piq.write_jsonl(specs, tmp_path / f"{setting}.jsonl")
        loaded = load_specs(f)
        assert len(loaded) == 3 and loaded[0].num_steps == 50 and loaded[0].sigma_max == 80.0
    assert loaded[0].condition_frame_indexes_vision == list(range(19)) and loaded[0].num_frames == 193
    frames = np.zeros((193, 4, 4, 3), np.uint8)
    assert piq.scored_frames(frames, "v2v").shape[0] == 120
    assert piq.scored_frames(frames[:121], "i2v").shape[0] == 120
    cmd = piq.inference_command("s.jsonl", "out", gpus=4)
    assert "--cp-size=4" in cmd and "--no-guardrails" in cmd


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
def test_preview_helpers_on_reference_specs(tmp_path):
    from cosmos_b200.utils import preview_helpers as ph

    d = REF / "cookbooks/cosmos3/generator/transfer/specs"
    spec = ph.load_transfer_spec("depth", d)
    assert spec["depth"]["control_path"].endswith("control_depth.mp4")
    assert ph.resolve_spec_path(spec["prompt_path"], d).name == "prompt.json"
    with pytest.raises(ValueError):
        ph.load_transfer_spec("nope", d)
    yy, xx = np.mgrid[0:32, 0:48]
    clip = np.repeat(np.stack([xx * 4, yy * 6, xx + yy], -1).astype(np.uint8)[None], 3, 0)
    src = tmp_path / "vision.mp4"
    mp4.write_mp4_mjpeg(src, clip, 10)
    prev = ph.make_preview(src)
    assert prev.exists() and prev.name == "vision_preview.mp4"


def test_truncated_and_damaged_spec_files_are_reported_not_half_read(tmp_path):
    """Host-side fault injection on the input side: a spec cut off mid-write, a JSONL with one damaged line, an
    empty file and a non-object sample all stop the run with a message that names the file (and the line)."""
    good = {"model_mode": "text2video", "name": "a", "prompt": "p", "resolution": "256", "num_frames": 5}
    whole = json.dumps(good)
    cut = tmp_path / "cut.json"
    cut.write_text(whole[:len(whole) // 2])
    with pytest.raises(SpecError, match=r"cut\.json: invalid JSON"):
        load_specs(cut)
    lines = tmp_path / "batch.jsonl"
    lines.write_text(whole + "\n\n" + whole.replace('"a"', '"b"')[:-7] + "\n" + whole.replace('"a"', '"c"') + "\n")
    with pytest.raises(SpecError, match=r"batch\.jsonl:3: invalid JSON"):
        load_specs(lines)
    empty = tmp_path / "empty.jsonl"
    empty.write_text("\n\n")
    with pytest.raises(SpecError, match="no samples"):
        load_specs(empty)
    arr = tmp_path / "arr.json"
    arr.write_text("[1, 2]")
    with pytest.raises(SpecError, match="must be a JSON object"):
        load_specs(arr)
    with pytest.raises(SpecError, match="not found"):
        load_specs(tmp_path / "missing.json")


def test_foreign_codecs_are_decoded_through_opencv_with_seeking(tmp_path):
    """A clip that is not this package's own Motion-JPEG layout (here MPEG-4 part 2 written by OpenCV) goes through
    OpenCV's decoders; `start` seeks instead of decoding from the beginning."""
    cv2 = pytest.importorskip("cv2")
    from cosmos_b200.io import media
    path = tmp_path / "clip.mp4"
    w = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"mp4v"), 12.0, (96, 64))
    if not w.isOpened():
        pytest.skip("this OpenCV build has no MPEG-4 encoder")
    for t in range(20):
        frame = np.full((64, 96, 3), 16, dtype=np.uint8)
        frame[:, 4 * t:4 * t + 8] = (0, 0, 255)             # BGR: a red bar that moves right
        w.write(frame)
    w.release()
    frames, fps = media.read_video(path)
    assert frames.shape == (20, 64, 96, 3) and abs(fps - 12.0) < 1e-3
    red = frames[..., 0].astype(int) - frames[..., 2].astype(int)
    cols = [int(red[t].mean(0).argmax()) for t in range(20)]
    assert all(4 * t <= cols[t] < 4 * t + 8 for t in range(20))                       # RGB order, frame order
    tail, _ = media.read_video(path, max_frames=3, start=15)
    assert tail.shape[0] == 3 and np.abs(tail.astype(int) - frames[15:18].astype(int)).max() <= 2
    small, _ = media.read_video(path, max_frames=2, size=(48, 32))
    assert small.shape == (2, 32, 48, 3)


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
def test_droid_lerobot_dataset_items_carry_the_decoded_views():
    pytest.importorskip("cv2")
    from cosmos_b200.data.vfm.action.datasets import DROIDLeRobotDataset

    root = REF / "cookbooks/cosmos3/generator/action/assets/droid_lerobot_example"
    ds = DROIDLeRobotDataset(root, action_chunk_size=16)
    a, b = ds[0], ds[3]
    assert a["video"].shape[:2] == (3, 17) and a["video"].shape[2] == 360 and a["video"].shape[3] % 640 == 0
    assert a["video"].dtype == np.uint8 and b["frame_index"] == 48
    assert np.abs(a["video"].astype(int) - b["video"].astype(int)).mean() > 0.1      # another part of the episode


def test_sample_video_keeps_only_the_sampled_frames(tmp_path):
    from cosmos_b200.io import media
    frames = np.zeros((30, 32, 48, 3), dtype=np.uint8)
    for t in range(30):
        frames[t, :, :, 1] = 8 * t                                   # the green level tells the frame apart
    clip = tmp_path / "own.mp4"
    media.write_video(clip, frames, 10, 8, None, 48000)              # this package's Motion-JPEG layout
    got, times, fps = media.sample_video(clip, fps=2.0)
    assert abs(fps - 10.0) < 1e-6 and got.shape == (6, 32, 48, 3) and times == pytest.approx([0.0, 0.5, 1.0, 1.5, 2.0, 2.5])
    assert [int(round(g[..., 1].mean() / 8)) for g in got] == [0, 5, 10, 15, 20, 25]
    got, times, _ = media.sample_video(clip, num_frames=4)
    assert [int(round(g[..., 1].mean() / 8)) for g in got] == [0, 10, 19, 29] and times[-1] == pytest.approx(2.9)
    got, times, _ = media.sample_video(clip, limit=7)
    assert got.shape[0] == 7 and times[1] == pytest.approx(0.1)
    np.save(tmp_path / "arr.npy", frames)                            # arrays go through the in-memory path
    got, times, fps = media.sample_video(tmp_path / "arr.npy", fps=12.0)
    assert fps == 24.0 and got.shape[0] == 15 and times[1] == pytest.approx(2 / 24)


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
@pytest.mark.parametrize("control", ["edge", "depth"])
def test_reference_transfer_specs_run_with_their_own_assets(control, tmp_path):
    """The reference's transfer specs as they are (prompt JSON files, H.264 control clips, chunking keys), shrunk
    only in size and steps, through the CLI's sample runner on the tiny model."""
    pytest.importorskip("cv2")
    import dataclasses

    import torch
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    from cosmos_b200.scripts import inference as cli

    spec = load_specs(REF / "cookbooks/cosmos3/generator/transfer/specs" / f"{control}.json")[0]
    assert spec.is_transfer and control in spec.controls and spec.prompt_path and spec.negative_prompt_file
    spec = dataclasses.replace(spec, resolution="256", num_frames=9, num_steps=1, num_video_frames_per_chunk=9)
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=32, n_layers=1))
    with pytest.warns(UserWarning, match="truncated to max_sequence_length"):       # dense JSON prompt, byte tokenizer
        rec = cli.run_generator_sample(pipe, spec, tmp_path / control, 8, True)
    assert rec["model_mode"] == "video2video" and (tmp_path / control / "vision.mp4").stat().st_size > 1000
    from cosmos_b200.io import media
    frames, fps = media.read_video(tmp_path / control / "vision.mp4")
    assert frames.shape[0] == 9 and abs(fps - spec.fps) < 1e-6


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
def test_action_modes_run_on_the_reference_action_assets(tmp_path):
    """Forward dynamics from the reference's AV trajectory (60 x 9) and start image, inverse dynamics on its UMI
    clip (H.264): spec files as the notebooks write them, shrunk in size and steps, on the tiny model."""
    pytest.importorskip("cv2")
    import torch
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    from cosmos_b200.scripts import inference as cli

    assets = REF / "cookbooks/cosmos3/generator/action/assets"
    fd = {"model_mode": "forward_dynamics", "name": "av_forward", "prompt": "drive forward", "vision_path": str(assets / "images/av_0.jpg"),
          "action_path": str(assets / "actions/av_traj_forward.json"), "action_chunk_size": 8, "domain_name": "av",
          "image_size": 256, "view_point": "ego_view", "num_steps": 1, "guidance": 1.0}
    idn = {"model_mode": "inverse_dynamics", "name": "umi_id", "prompt": "", "vision_path": str(assets / "videos/umi.mp4"),
           "action_chunk_size": 8, "domain_name": "umi", "image_size": 256, "num_steps": 1, "guidance": 1.0}
    (tmp_path / "specs.jsonl").write_text(json.dumps(fd) + "\n" + json.dumps(idn) + "\n")
    specs = load_specs(tmp_path / "specs.jsonl")
    assert [s.num_frames for s in specs] == [9, 9] and specs[0].fps == 10 and specs[1].fps == 20      # chunk + 1; domain fps
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=16, n_layers=1))
    rec = cli.run_generator_sample(pipe, specs[0], tmp_path / "fd", 8, True)
    assert rec["model_mode"] == "forward_dynamics" and (tmp_path / "fd" / "vision.mp4").stat().st_size > 1000
    rec = cli.run_generator_sample(pipe, specs[1], tmp_path / "id", 8, True)
    out = json.loads((tmp_path / "id" / "sample_outputs.json").read_text())
    act = np.asarray(out["outputs"][0]["content"]["action"])
    assert act.shape == (8, 10) and np.isfinite(act).all()                                              # UMI: 9-D pose + gripper


def test_action_normalizer_standardises_free_dims_and_travels_with_the_checkpoint(tmp_path):
    import torch
    from cosmos_b200.data.vfm.action.normalization import ActionNormalizer, default_free_dims
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    rng = np.random.default_rng(0)
    chunks = [np.concatenate([rng.normal(0.02, 0.01, (16, 3)), rng.normal(0, 1, (16, 6)), rng.uniform(0, 1, (16, 1))], -1)
              for _ in range(20)]
    assert list(default_free_dims(10)) == [0, 1, 2, 9] and list(default_free_dims(9)) == [0, 1, 2]
    norm = ActionNormalizer()
    assert np.array_equal(norm.normalize(chunks[0], "droid_lerobot"), chunks[0].astype(np.float32))      # no statistics: identity
    norm.fit("droid_lerobot", chunks)
    z = norm.normalize(np.concatenate(chunks), "droid_lerobot")
    assert np.abs(z[:, [0, 1, 2, 9]].mean(0)).max() < 1e-3 and np.abs(z[:, [0, 1, 2, 9]].std(0) - 1).max() < 1e-3
    assert np.allclose(z[:, 3:9], np.concatenate(chunks)[:, 3:9], atol=1e-6)                            # rot6d untouched
    assert np.allclose(norm.denormalize(z, "droid_lerobot"), np.concatenate(chunks), atol=1e-5)
    with pytest.raises(ValueError):
        norm.normalize(np.zeros((4, 9)), "droid_lerobot")
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=16, n_layers=1))
    pipe.action_normalizer = norm
    pipe.save_pretrained(tmp_path / "ckpt")
    again = Cosmos3OmniPipeline.from_pretrained(str(tmp_path / "ckpt"), torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16))
    assert again.action_normalizer.stats == norm.stats
    # inverse dynamics output comes back in the data's units: the gripper column is mean + std * z
    dom = list(again.cfg.action_domains).index("droid_lerobot")
    clip = (rng.random((5, 32, 32, 3)) * 255).astype(np.uint8)
    kw = dict(prompt="", video=clip, num_frames=5, height=32, width=32, num_inference_steps=1, guidance_scale=1.0, domain=dom,
              action_dim=10, n_action=4, denoise_action=True, output_type="np")
    got = again(generator=torch.Generator().manual_seed(1), **kw).action
    again.action_normalizer = None
    raw = again(generator=torch.Generator().manual_seed(1), **kw).action
    assert got.shape == raw.shape == (4, 10) and np.allclose(got, norm.denormalize(raw, "droid_lerobot"), atol=1e-5)

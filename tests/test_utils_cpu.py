"""Small contracts of utility modules: prompt upsampler fallback and schema keys, AV domain constants,
phase timer / JSONL logger, CUDA-graph wrapper (GPU only)."""
import json

import pytest
import torch


def test_prompt_upsampler_returns_compact_json_with_template_fields():
    from cosmos_b200.config import DecodingConfig, tiny_config
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.models.reasoner import ReasonerEngine
    from cosmos_b200.utils import prompt_upsampler as pu
    from cosmos_b200.utils.tokenizer import load_tokenizer

    assert pu.UPSAMPLER_DECODING.seed == 3407 and pu.UPSAMPLER_DECODING.presence_penalty == 1.5
    assert {"subjects", "lighting", "cinematography", "actions", "audio_description"} <= set(pu.TOP_LEVEL_KEYS)
    cfg = tiny_config(n_layers=1)
    model = MoTModel(cfg, dtype=torch.float32, device="cpu")
    model.init_weights(seed=2)
    tok = load_tokenizer(None, cfg.vocab_size)
    out = pu.upsample_prompt(ReasonerEngine(model), tok, "a cat jumps", 1280, 720, 5.0, 24,
                             decoding=DecodingConfig(max_new_tokens=4, do_sample=False))
    obj = json.loads(out)                                   # random weights: the fallback wraps the raw prompt
    assert obj["temporal_caption"] == "a cat jumps" and obj["resolution"] == {"W": 1280, "H": 720}
    assert obj["fps"] == 24 and obj["duration"] == 5.0 and ": " not in out


def test_av_domain_constants_match_the_action_conventions():
    from cosmos_b200.data.vfm.action import av_dataset as av
    from cosmos_b200.io.spec import DOMAINS

    assert (av.AV_ROTATION_FORMAT, av.AV_POSE_CONVENTION, av.AV_TRANSLATION_SCALE) == ("rot6d", "backward_framewise", 1.35)
    assert av.DOMAIN_ACTION_DIM["av"] == 9 and av.DOMAIN_ACTION_DIM["droid_lerobot"] == 10
    assert set(DOMAINS) <= set(av.DOMAIN_ACTION_DIM)
    assert av.DOMAIN_DEFAULTS["av"]["action_chunk_size"] == 60 and av.DOMAIN_DEFAULTS["umi"]["image_size"] == 256


def test_phase_timer_and_jsonl_logger(tmp_path):
    from cosmos_b200.utils.obs import JsonlLogger, PhaseTimer, write_benchmark_json

    t = PhaseTimer()
    with t.phase("a"):
        torch.randn(64, 64) @ torch.randn(64, 64)
    with t.phase("a"):
        pass
    with t.phase("b"):
        pass
    s = t.summary_ms()
    assert set(s) == {"a", "b"} and s["a"] >= 0
    log = JsonlLogger(str(tmp_path / "log.jsonl"), stdout=False)
    log.log(step=1, loss=0.5)
    log.log(step=2, loss=0.25)
    rows = [json.loads(line) for line in (tmp_path / "log.jsonl").read_text().splitlines()]
    assert [r["step"] for r in rows] == [1, 2] and "ts" in rows[0]
    p = write_benchmark_json(tmp_path, [{"generation_time_s": 2.0}, {"generation_time_s": 4.0}])
    assert json.loads(p.read_text())["average"]["generation_time_s"] == 3.0


@pytest.mark.gpu
def test_graphed_callable_replays_with_new_inputs():
    from cosmos_b200.utils.graphs import GraphedCallable

    w = torch.randn(64, 64, device="cuda")
    g = GraphedCallable(lambda x: torch.relu(x @ w), [torch.randn(8, 64, device="cuda")])
    for _ in range(3):
        x = torch.randn(8, 64, device="cuda")
        torch.testing.assert_close(g(x), torch.relu(x @ w))


def test_media_helpers_follow_the_diffusers_call_shapes(tmp_path):
    import numpy as np
    from PIL import Image

    from cosmos_b200.io import media
    from cosmos_b200.utils.media_helpers import encode_video, export_to_video, load_image
    frames = (np.random.rand(6, 32, 48, 3) * 255).astype(np.uint8)
    p = export_to_video(frames, str(tmp_path / "a.mp4"), fps=12, macro_block_size=1)
    back, fps = media.read_video(p)
    assert back.shape == frames.shape and abs(fps - 12) < 1e-6
    pil = [Image.fromarray(f) for f in frames]
    sound = np.stack([np.sin(np.linspace(0, 40, 24000)), np.zeros(24000)], axis=0).astype(np.float32)      # [2, N]
    q = encode_video(pil, fps=12, output_path=str(tmp_path / "b.mp4"), audio=sound, audio_sample_rate=48000)
    assert media.read_video(q)[0].shape == frames.shape and (tmp_path / "b.mp4").stat().st_size > (tmp_path / "a.mp4").stat().st_size
    floats = export_to_video(frames.astype(np.float32) / 255.0, tmp_path / "c.mp4", fps=8)
    assert np.abs(media.read_video(floats)[0].astype(int) - back.astype(int)).max() <= 2
    Image.fromarray(frames[0]).save(tmp_path / "i.png")
    img = load_image(tmp_path / "i.png")
    assert img.size == (48, 32) and img.mode == "RGB" and load_image(img).size == (48, 32)
    import pytest
    with pytest.raises(ValueError):
        load_image("https://example.com/x.png")


def test_top_level_package_exposes_the_public_classes_lazily():
    import importlib
    import sys

    import cosmos_b200
    assert cosmos_b200.__version__ == "0.1.0"
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    assert cosmos_b200.Cosmos3OmniPipeline is Cosmos3OmniPipeline
    assert cosmos_b200.Cosmos3ReasonerForConditionalGeneration.__name__ == "Cosmos3ReasonerForConditionalGeneration"
    assert cosmos_b200.SamplingConfig().num_steps == 35 and "UniPCMultistepScheduler" in dir(cosmos_b200)
    import pytest
    with pytest.raises(AttributeError):
        cosmos_b200.NoSuchThing
    assert importlib.import_module("cosmos_b200.ops") is sys.modules["cosmos_b200.ops"]      # submodules still import


def test_prompt_upsampler_cli_prints_a_compact_json_caption(capsys):
    import json

    from cosmos_b200.utils import prompt_upsampler as pu
    assert pu.main(["a robot arm stacks blocks", "--checkpoint-path", "tiny", "--resolution", "256", "--num-frames", "49",
                    "--fps", "24", "--max-tokens", "4", "--device", "cpu"]) == 0
    out = capsys.readouterr().out.strip().splitlines()[-1]
    obj = json.loads(out)
    assert obj["resolution"] == {"W": 320, "H": 192} and obj["fps"] == 24 and " " not in out.split('"temporal_caption"')[0]
    assert obj["temporal_caption"] == "a robot arm stacks blocks"          # random weights: the raw prompt is wrapped

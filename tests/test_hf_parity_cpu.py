"""Parity with the `transformers` implementation of Qwen3-VL, which the reference's Reasoner is based on: with the
same weights the AR tower gives the text model's hidden states (text-only, 3-D positions of an image grid, DeepStack
injection), the position-id builder gives `get_rope_index`'s ids, and the vision encoder gives the vision model's
merged embeddings and DeepStack features."""
import pytest
import torch

hfm = pytest.importorskip("transformers.models.qwen3_vl.modeling_qwen3_vl")
hfc = pytest.importorskip("transformers.models.qwen3_vl.configuration_qwen3_vl")

from cosmos_b200 import ops  # noqa: E402
from cosmos_b200.ckpt import hf_qwen3vl as hq  # noqa: E402
from cosmos_b200.config import tiny_config  # noqa: E402
from cosmos_b200.models.mot import MoTModel  # noqa: E402
from cosmos_b200.models.reasoner import ReasonerEngine  # noqa: E402
from cosmos_b200.models.vit import VisionEncoder  # noqa: E402

TEXT = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
            rope_parameters={"rope_type": "default", "rope_theta": 500000.0, "mrope_section": [3, 3, 2], "mrope_interleaved": True})
VISION = dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, patch_size=16, spatial_merge_size=2,
              temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=36, deepstack_visual_indexes=[0, 2])


def _randomise(module):
    torch.manual_seed(0)
    for n, p in module.named_parameters():
        torch.nn.init.normal_(p, 1.0 if ("norm" in n and n.endswith("weight")) else 0.0, 0.1 if "norm" in n else 0.05)


def _pair():
    hf = hfm.Qwen3VLTextModel(hfc.Qwen3VLTextConfig(**TEXT)).eval()
    _randomise(hf)
    cfg = tiny_config(**hq.config_kwargs_from_hf(hf.config))
    ours = MoTModel(cfg, dtype=torch.float32, device="cpu", towers=("ar",))
    hq.load_text_weights(ours, hf.state_dict())
    return hf, ours, cfg


def _hidden(ours, cfg, emb, pos, **kw):
    h, _ = ours.ar_forward(emb, pos, **kw)
    return ops.rmsnorm(h, ours.ar_norm, cfg.rms_eps)[0]


def test_ar_tower_reproduces_the_qwen3vl_text_model():
    hf, ours, cfg = _pair()
    assert (cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn_dim, cfg.mrope_section) == (64, 4, 2, 16, 128, (3, 3, 2))
    ids = torch.randint(0, 300, (1, 11))
    from cosmos_b200.models import rope
    with torch.no_grad():
        want = hf(input_ids=ids).last_hidden_state
        got = _hidden(ours, cfg, ours.embed_tokens(ids), rope.text_positions(11))
    assert (got - want).abs().max() < 2e-5
    # an image grid in the prompt: 3-D rotary ids, vision rows spliced in, DeepStack features after the first layers
    ids = torch.tensor([[5, 6, 292] + [290] * 6 + [293, 7, 8, 9]])
    vmask = ids == 290
    pos = ReasonerEngine.positions(ReasonerEngine.__new__(ReasonerEngine), ids, vmask, [(1, 2, 3)])
    emb = ours.embed_tokens(ids).clone()
    emb[vmask] = torch.randn(6, 64)
    deep = [torch.randn(6, 64), torch.randn(6, 64)]
    with torch.no_grad():
        want = hf(inputs_embeds=emb, position_ids=pos[:, None], visual_pos_masks=vmask, deepstack_visual_embeds=deep).last_hidden_state
        got = _hidden(ours, cfg, emb, pos, deepstack=deep, vision_mask=vmask)
        plain = _hidden(ours, cfg, emb, pos)
    assert (got - want).abs().max() < 2e-5 and (plain - want).abs().max() > 1e-2      # DeepStack matters and matches
    # export is the inverse of load
    back = hq.export_text_weights(ours, prefix="")
    sd = hf.state_dict()
    assert all(torch.equal(back[k], sd[k]) for k in sd) and torch.equal(back["lm_head.weight"], sd["embed_tokens.weight"])


def test_position_ids_match_get_rope_index():
    cfg = hfc.Qwen3VLConfig(text_config=TEXT, vision_config=VISION, image_token_id=290, video_token_id=291,
                            vision_start_token_id=292, vision_end_token_id=293)
    hf = hfm.Qwen3VLModel(cfg).eval()
    eng = ReasonerEngine.__new__(ReasonerEngine)
    ids = torch.tensor([[5, 6, 292] + [290] * 6 + [293, 7, 292] + [290] * 4 + [293, 9]])
    want, _ = hf.get_rope_index(ids, (ids == 290).int(), image_grid_thw=torch.tensor([[1, 4, 6], [1, 4, 4]]))
    assert torch.equal(ReasonerEngine.positions(eng, ids, ids == 290, [(1, 2, 3), (1, 2, 2)]), want[:, 0])
    # a clip is laid out frame group by frame group, each in its own vision_start / vision_end pair
    ids = torch.tensor([[5, 292] + [291] * 6 + [293, 292] + [291] * 6 + [293, 7, 8]])
    want, _ = hf.get_rope_index(ids, (ids == 291).int() * 2, video_grid_thw=torch.tensor([[2, 4, 6]]))
    assert torch.equal(ReasonerEngine.positions(eng, ids, ids == 291, [(1, 2, 3), (1, 2, 3)]), want[:, 0])


@pytest.mark.parametrize("frames,height,width", [(1, 64, 96), (4, 96, 64), (3, 160, 192)])
def test_vision_encoder_reproduces_the_qwen3vl_vision_model(frames, height, width):
    hv = hfm.Qwen3VLVisionModel(hfc.Qwen3VLVisionConfig(**VISION)).eval()
    _randomise(hv)
    cfg = tiny_config(d_model=64, **{k: v for k, v in hq.config_kwargs_from_hf(hfc.Qwen3VLTextConfig(**TEXT), hv.config).items()
                                     if k.startswith("vit_")})
    assert (cfg.vit_depth, cfg.vit_hidden, cfg.vit_ffn, cfg.vit_pos_side, cfg.vit_deepstack) == (3, 32, 48, 6, (0, 2))
    vit = VisionEncoder(cfg).eval()
    hq.load_vision_weights(vit, hv.state_dict())
    torch.manual_seed(1)
    video = torch.rand(frames, 3, height, width) * 2 - 1
    pixels = hq.hf_image_patches(video, 16, 2, 2)
    t = (frames + 1) // 2
    with torch.no_grad():
        out = hv(pixels, grid_thw=torch.tensor([[t, height // 16, width // 16]]))
        got, grid, deep = vit(video, return_deepstack=True)
    want = out.pooler_output if hasattr(out, "pooler_output") else out[0]
    want_deep = out.deepstack_features if hasattr(out, "deepstack_features") else out[1]
    assert grid == (t, height // 32, width // 32) and got.shape == want.shape
    assert (got - want).abs().max() < 5e-5, float((got - want).abs().max())
    assert len(deep) == len(want_deep) == 2
    for a, b in zip(deep, want_deep):
        assert (a - b).abs().max() < 5e-5


def test_reasoner_class_loads_a_qwen3vl_checkpoint_directory(tmp_path):
    """save_pretrained of a (tiny) Qwen3VLForConditionalGeneration -> our Reasoner class reads config and safetensors,
    gives the same next-token logits for text and for a prompt with an image, and exports the text tower back."""
    from cosmos_b200.hf import Cosmos3ReasonerForConditionalGeneration
    cfg = hfc.Qwen3VLConfig(text_config=TEXT, vision_config=VISION, image_token_id=290, video_token_id=291,
                            vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False)
    hf = hfm.Qwen3VLForConditionalGeneration(cfg).eval()
    _randomise(hf)
    hf.save_pretrained(tmp_path / "qwen", safe_serialization=True)
    ours = Cosmos3ReasonerForConditionalGeneration.from_pretrained(str(tmp_path / "qwen"))
    mc = ours.model.cfg
    assert (mc.d_model, mc.n_layers, mc.vit_depth, mc.vit_deepstack, mc.mrope_section) == (64, 2, 3, (0, 2), (3, 3, 2))
    ids = torch.randint(0, 280, (1, 9))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = ours(ids)
    assert (got - want).abs().max() < 5e-5
    # prompt with one 64 x 96 image: 2 x 3 merged tokens
    video = torch.rand(1, 3, 64, 96) * 2 - 1
    ids = torch.tensor([[5, 6, 292] + [290] * 6 + [293, 7, 8, 9]])
    pixels = hq.hf_image_patches(video, 16, 2, 2)
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=torch.tensor([[1, 4, 6]]),
                  mm_token_type_ids=(ids == 290).int()).logits[0, -1]
        eng = ReasonerEngine(ours.model, ours.visual)
        emb, grid, deep = ours.visual(video, return_deepstack=True)
        vmask = ids == 290
        logits, _ = eng.prefill(eng.embed(ids, emb, vmask), eng.positions(ids, vmask, [grid]), deep, vmask)
    assert (logits[0] - want).abs().max() < 1e-4 and int(logits[0].argmax()) == int(want.argmax())
    ours.save_qwen3vl(tmp_path / "export")
    from cosmos_b200.ckpt import safetensors_io as sio
    files = sio.tensor_files(tmp_path / "export")
    key = "model.language_model.layers.1.mlp.down_proj.weight"
    assert key in files and torch.equal(sio.open_reader(files[key]).get(key), hf.state_dict()[key])


def test_exported_reasoner_loads_in_transformers_and_gives_the_same_logits(tmp_path):
    """The other direction: a Reasoner of this framework (random weights) saved in the Qwen3-VL layout is loaded by
    `transformers` itself and agrees on text and on an image prompt."""
    from cosmos_b200.hf import Cosmos3ReasonerConfig, Cosmos3ReasonerForConditionalGeneration
    over = dict(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_dim=96, vocab_size=320, mrope_section=[3, 3, 2],
                vit_depth=2, vit_hidden=32, vit_heads=2, vit_ffn=40, vit_pos_side=5, vit_deepstack=[1])
    ours = Cosmos3ReasonerForConditionalGeneration(Cosmos3ReasonerConfig("tiny", over)).eval()
    _randomise(ours.visual)
    ours.save_qwen3vl(tmp_path / "out", dict(image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293))
    hf = hfm.Qwen3VLForConditionalGeneration.from_pretrained(str(tmp_path / "out"), torch_dtype=torch.float32).eval()
    ids = torch.randint(0, 280, (1, 7))
    with torch.no_grad():
        assert (hf(input_ids=ids).logits - ours(ids)).abs().max() < 5e-5
    video = torch.rand(2, 3, 96, 64) * 2 - 1
    ids = torch.tensor([[9, 292] + [290] * 6 + [293, 4, 3]])
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=hq.hf_image_patches(video, 16, 2, 2), image_grid_thw=torch.tensor([[1, 6, 4]]),
                  mm_token_type_ids=(ids == 290).int()).logits[0, -1]
        eng = ReasonerEngine(ours.model, ours.visual)
        emb, grid, deep = ours.visual(video, return_deepstack=True)
        vmask = ids == 290
        logits, _ = eng.prefill(eng.embed(ids, emb, vmask), eng.positions(ids, vmask, [grid]), deep, vmask)
    assert grid == (1, 3, 2) and (logits[0] - want).abs().max() < 1e-4


def test_generate_takes_processor_style_patch_rows(tmp_path):
    """Greedy continuation of a two-image prompt: our class fed with `transformers`-processor inputs (patch rows +
    image_grid_thw) produces the tokens `transformers`' own generate produces from the same checkpoint."""
    from cosmos_b200.hf import Cosmos3ReasonerForConditionalGeneration
    cfg = hfc.Qwen3VLConfig(text_config=TEXT, vision_config=VISION, image_token_id=290, video_token_id=291,
                            vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False)
    hf = hfm.Qwen3VLForConditionalGeneration(cfg).eval()
    _randomise(hf)
    hf.save_pretrained(tmp_path / "qwen", safe_serialization=True)
    ours = Cosmos3ReasonerForConditionalGeneration.from_pretrained(str(tmp_path / "qwen"))
    a, b = torch.rand(1, 3, 64, 96) * 2 - 1, torch.rand(1, 3, 64, 64) * 2 - 1
    pixels = torch.cat([hq.hf_image_patches(a, 16, 2, 2), hq.hf_image_patches(b, 16, 2, 2)])
    grids = torch.tensor([[1, 4, 6], [1, 4, 4]])
    assert torch.allclose(hq.frames_from_hf_patches(pixels[:24], grids[0], 16, 2, 2)[:1], a)       # the inverse layout map
    ids = torch.tensor([[5, 292] + [290] * 6 + [293, 7, 292] + [290] * 4 + [293, 8, 9]])
    with torch.no_grad():                                     # teacher-forced logits of the whole prompt
        full = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grids, mm_token_type_ids=(ids == 290).int()).logits
        assert (ours(ids, pixel_values=pixels, image_grid_thw=grids, image_token_id=290) - full).abs().max() < 1e-4
    got = ours.generate(ids, pixel_values=pixels, image_grid_thw=grids, image_token_id=290, max_new_tokens=5)
    with torch.no_grad():
        want = hf.generate(input_ids=ids, pixel_values=pixels, image_grid_thw=grids, mm_token_type_ids=(ids == 290).int(),
                           attention_mask=torch.ones_like(ids), max_new_tokens=5, do_sample=False, eos_token_id=None, pad_token_id=0)
    assert got.shape == (1, ids.shape[1] + 5) and torch.equal(got, want)


def test_pipeline_opens_a_qwen3vl_directory_as_a_reasoner_only_checkpoint(tmp_path):
    """`--checkpoint-path <Qwen3-VL dir>`: AR tower and vision encoder come from the checkpoint (no DM tower is built),
    the server answers a chat with an image from it, and save_pretrained / from_pretrained keep the vision encoder."""
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    cfg = hfc.Qwen3VLConfig(text_config=TEXT, vision_config=VISION, image_token_id=290, video_token_id=291,
                            vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False)
    hf = hfm.Qwen3VLForConditionalGeneration(cfg).eval()
    _randomise(hf)
    hf.save_pretrained(tmp_path / "qwen", safe_serialization=True)
    pipe = Cosmos3OmniPipeline.from_pretrained(str(tmp_path / "qwen"), torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16))
    assert pipe.transformer.has_ar and not hasattr(pipe.transformer, "dm") and pipe.cfg.vit_deepstack == (0, 2)
    vit = pipe.vision_encoder()
    assert vit is pipe.vision_encoder()                                           # built once
    sd = hf.state_dict()
    assert torch.equal(vit.pos, sd["model.visual.pos_embed.weight"])
    assert torch.equal(pipe.transformer.embed, sd["model.language_model.embed_tokens.weight"])
    eng = ReasonerEngine(pipe.transformer, vit)
    from cosmos_b200.config import DecodingConfig
    ids = [5, 6, 7, 8, 9, 10]
    new, _ = eng.generate(ids, DecodingConfig(max_new_tokens=4, do_sample=False, presence_penalty=0.0), ())
    with torch.no_grad():
        want = hf.generate(input_ids=torch.tensor([ids]), attention_mask=torch.ones(1, 6, dtype=torch.long), max_new_tokens=4,
                           do_sample=False, eos_token_id=None, pad_token_id=0)
    assert new == want[0, 6:].tolist()
    pipe.save_pretrained(tmp_path / "ours")
    again = Cosmos3OmniPipeline.from_pretrained(str(tmp_path / "ours"), torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                                towers=("ar",))
    assert torch.equal(again.vision_encoder().pos, vit.pos) and torch.equal(again.transformer.embed, pipe.transformer.embed)


def test_video_prompt_layout_follows_the_qwen3vl_processor():
    """Clips enter the prompt as one vision segment per temporal group behind a "<t seconds>" stamp; the stamps are
    the processor's (`_calculate_timestamps`) and the rotary ids of that layout are `get_rope_index`'s."""
    from transformers.models.qwen3_vl.processing_qwen3_vl import Qwen3VLProcessor
    from cosmos_b200.utils.tokenizer import ByteTokenizer, video_layout
    idx, fps = [0, 6, 12, 18, 24], 24.0                                  # five sampled frames of a 24 fps clip
    want = Qwen3VLProcessor._calculate_timestamps(None, list(idx), fps, 2)
    lay = video_layout((3, 2, 3), [i / fps for i in idx], temporal_patch=2)
    assert lay["per_frame"] == 6 and lay["timestamps"] == pytest.approx(want) and len(want) == 3
    tok = ByteTokenizer(512)
    ids = tok.apply_chat_template([{"role": "user", "content": [{"type": "video_url"}, {"type": "text", "text": "what happens?"}]}],
                                  True, [lay])
    text = tok.decode(ids, skip_special=False)
    assert text.count("<|vision_start|>") == 3 and ids.count(tok.video_pad_id) == 18
    assert "<0.1 seconds><|vision_start|>" in text and "<0.6 seconds><|vision_start|>" in text and "<1.0 seconds><|vision_start|>" in text
    # the same token pattern in the checkpoint's id space: positions agree with the reference implementation
    cfg = hfc.Qwen3VLConfig(text_config=TEXT, vision_config=VISION, image_token_id=290, video_token_id=291,
                            vision_start_token_id=292, vision_end_token_id=293)
    hf = hfm.Qwen3VLModel(cfg).eval()
    seq = [5]
    for _ in range(3):
        seq += [11, 12, 292] + [291] * 6 + [293]                         # stamp tokens, then the segment
    seq += [7, 8]
    t = torch.tensor([seq])
    want_pos, _ = hf.get_rope_index(t, (t == 291).int() * 2, video_grid_thw=torch.tensor([[3, 4, 6]]))
    got = ReasonerEngine.positions(ReasonerEngine.__new__(ReasonerEngine), t, t == 291, [(1, 2, 3)] * 3)
    assert torch.equal(got, want_pos[:, 0])


def test_cli_runs_a_reasoner_sample_on_a_qwen3vl_directory_with_its_tokenizer(tmp_path):
    """The inference CLI pointed at a Qwen3-VL checkpoint directory (weights + tokenizer files): the checkpoint's
    tokenizer builds the chat prompt, the image goes through the checkpoint's vision tower, the text lands in
    reasoner_text.txt."""
    import json

    import numpy as np
    from PIL import Image

    from cosmos_b200.scripts import inference as cli
    from cosmos_b200.utils.tokenizer import HFTokenizer
    from tests.test_tokenizer_cpu import _write_tokenizer
    cfg = hfc.Qwen3VLConfig(text_config=TEXT, vision_config=VISION, image_token_id=290, video_token_id=291,
                            vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False)
    hf = hfm.Qwen3VLForConditionalGeneration(cfg).eval()
    _randomise(hf)
    ckpt = tmp_path / "qwen"
    hf.save_pretrained(ckpt, safe_serialization=True)
    _write_tokenizer(ckpt)
    Image.fromarray((np.random.rand(64, 96, 3) * 255).astype(np.uint8)).save(tmp_path / "frame.png")
    (tmp_path / "spec.json").write_text(json.dumps({"name": "r1", "model_mode": "reasoner", "prompt": "what is this ?",
                                                    "vision_path": "frame.png", "enable_sound": False, "max_new_tokens": 4,
                                                    "do_sample": False}))
    rc = cli.main(["-i", str(tmp_path / "spec.json"), "-o", str(tmp_path / "out"), "--checkpoint-path", str(ckpt),
                   "--no-guardrails", "--benchmark", "--device", "cpu"])
    assert rc == 0
    text = (tmp_path / "out" / "r1" / "reasoner_text.txt").read_text()
    bench = json.loads((tmp_path / "out" / "benchmark.json").read_text())
    assert isinstance(text, str) and "average" in bench
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    pipe = Cosmos3OmniPipeline.from_pretrained(str(ckpt), torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16))
    assert isinstance(pipe.tokenizer, HFTokenizer) and pipe.tokenizer.image_pad_id < pipe.cfg.vocab_size

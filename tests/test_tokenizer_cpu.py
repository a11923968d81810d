"""Tokenizers: the byte-level stand-in and the adapter around a checkpoint's own tokenizer files (built here with
the `tokenizers` library, no download)."""
import json

import pytest

from cosmos_b200.utils.tokenizer import ByteTokenizer, HFTokenizer, load_tokenizer

SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>",
            "<|video_pad|>"]


def _write_tokenizer(d, specials=SPECIALS):
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    words = ["a", "robot", "arm", "lifts", "the", "red", "cube", "user", "assistant", "system", "what", "is", "this", "?"]
    vocab = {w: i for i, w in enumerate(["<unk>"] + words)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.decoder = decoders.Fuse()
    tok.add_special_tokens(specials)
    d.mkdir(parents=True, exist_ok=True)
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>",
                                                         "eos_token": "<|im_end|>", "pad_token": "<|endoftext|>"}))


def test_byte_tokenizer_round_trip_and_chat_layout():
    t = ByteTokenizer(512)
    ids = t.encode("héllo <|im_end|>")
    assert ids[-1] == t.eos_id and t.decode(ids) == "héllo " and t.decode(ids, skip_special=False).endswith("<|im_end|>")
    chat = t.apply_chat_template([{"role": "user", "content": [{"type": "image_url"}, {"type": "text", "text": "hi"}]}], True, [3])
    assert chat.count(t.image_pad_id) == 3 and t.decode(chat, skip_special=False).endswith("<|im_start|>assistant\n")
    assert t.pad_or_truncate([1, 2, 3], 5) == [1, 2, 3, t.pad_id, t.pad_id] and t.pad_or_truncate([1, 2, 3], 2) == [1, 2]


def test_checkpoint_tokenizer_is_used_through_the_adapter(tmp_path):
    _write_tokenizer(tmp_path / "ckpt" / "tokenizer")
    t = load_tokenizer(str(tmp_path / "ckpt"), 512)
    assert isinstance(t, HFTokenizer)
    ids = t.encode("a robot arm lifts the red cube")
    assert len(ids) == 7 and t.decode(ids).replace(" ", "") == "arobotarmliftstheredcube"
    assert len({t.eos_id, t.eot_id, t.image_pad_id, t.video_pad_id}) == 4 and t.pad_id == t.eot_id
    assert t.pad_or_truncate(ids, 9)[-2:] == [t.pad_id, t.pad_id]
    msgs = [{"role": "system", "content": "a robot"},
            {"role": "user", "content": [{"type": "video_url"}, {"type": "image_url"}, {"type": "text", "text": "what is this ?"}]}]
    chat = t.apply_chat_template(msgs, True, [4, 2])
    assert chat.count(t.video_pad_id) == 4 and chat.count(t.image_pad_id) == 2
    assert chat.count(t.special_ids["<|im_start|>"]) == 3 and chat.count(t.eos_id) == 2     # two turns + the open assistant turn
    v0 = chat.index(t.special_ids["<|vision_start|>"])
    assert chat[v0 + 1:v0 + 5] == [t.video_pad_id] * 4 and chat[v0 + 5] == t.special_ids["<|vision_end|>"]
    with pytest.raises(ValueError):
        t.apply_chat_template([{"role": "user", "content": [{"type": "audio"}]}])
    assert isinstance(load_tokenizer(str(tmp_path / "nothing"), 512), ByteTokenizer)


def test_adapter_names_missing_special_tokens(tmp_path):
    _write_tokenizer(tmp_path / "bad", specials=["<|endoftext|>", "<|im_start|>", "<|im_end|>"])
    with pytest.raises(ValueError, match="vision_start"):
        load_tokenizer(str(tmp_path / "bad"), 512)


def test_pipeline_and_reasoner_run_on_a_checkpoint_tokenizer(tmp_path):
    """save_pretrained + tokenizer files -> from_pretrained picks the checkpoint's tokenizer; generation and a chat
    prefill run through it."""
    import torch
    from cosmos_b200.config import DecodingConfig
    from cosmos_b200.models.reasoner import ReasonerEngine
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(n_layers=1, max_text_len=16))
    pipe.save_pretrained(tmp_path / "ckpt")
    _write_tokenizer(tmp_path / "ckpt" / "tokenizer")
    again = Cosmos3OmniPipeline.from_pretrained(str(tmp_path / "ckpt"), torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                                enable_safety_checker=False)
    assert isinstance(again.tokenizer, HFTokenizer)
    ids = again.encode_text("a robot arm lifts the red cube")
    assert ids.shape == (1, 16) and int(ids[0, 7]) == again.tokenizer.pad_id
    out = again(prompt="a robot arm", num_frames=1, height=32, width=32, num_inference_steps=1, guidance_scale=1.0)
    assert out.video[0].size == (32, 32)                       # a single image comes back as [PIL.Image] by default
    again.save_pretrained(tmp_path / "copy")
    assert (tmp_path / "copy" / "tokenizer" / "tokenizer.json").exists()
    assert isinstance(load_tokenizer(str(tmp_path / "copy"), 512), HFTokenizer)
    tok = again.tokenizer
    chat = tok.apply_chat_template([{"role": "user", "content": "what is this ?"}], True)
    eng = ReasonerEngine(again.transformer, None)
    new, usage = eng.generate(chat, DecodingConfig(max_new_tokens=3, do_sample=False), (tok.eos_id, tok.eot_id))
    assert 1 <= len(new) <= 3 and usage["prompt_tokens"] == len(chat)

"""Text tokenizers. A checkpoint directory that ships Hugging Face tokenizer files is loaded
through `transformers.AutoTokenizer`; otherwise (random-init / offline runs) a deterministic
byte-level tokenizer is used: ids 0..255 are UTF-8 bytes, followed by the special tokens.
The chat template mirrors the Qwen-style layout the reference's Reasoner uses
(`<|im_start|>role\\n...<|im_end|>`; reference cookbooks/cosmos3/reasoner/reasoner_prompt_guide.md:29-75).
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    SPECIALS = ["<|pad|>", "<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>",
                "<|image_pad|>", "<|video_pad|>", "<think>", "</think>", "<|bog|>"]

    def __init__(self, vocab_size: int = 32000):
        assert vocab_size >= 256 + len(self.SPECIALS)
        self.vocab_size = vocab_size
        self.special_ids: Dict[str, int] = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.pad_id = self.special_ids["<|pad|>"]
        self.eos_id = self.special_ids["<|im_end|>"]
        self.eot_id = self.special_ids["<|endoftext|>"]
        self.image_pad_id = self.special_ids["<|image_pad|>"]
        self.video_pad_id = self.special_ids["<|video_pad|>"]

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        i = 0
        while i < len(text):
            if text[i] == "<":
                hit = next((s for s in self.SPECIALS if text.startswith(s, i)), None)
                if hit:
                    ids.append(self.special_ids[hit])
                    i += len(hit)
                    continue
            ids.extend(text[i].encode("utf-8"))
            i += 1
        return ids

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        out = bytearray()
        parts: List[str] = []
        inv = {v: k for k, v in self.special_ids.items()}
        for t in ids:
            t = int(t)
            if t < 256:
                out.append(t)
            else:
                if out:
                    parts.append(out.decode("utf-8", errors="replace"))
                    out = bytearray()
                if not skip_special and t in inv:
                    parts.append(inv[t])
        if out:
            parts.append(out.decode("utf-8", errors="replace"))
        return "".join(parts)

    def pad_or_truncate(self, ids: List[int], length: int) -> List[int]:
        """Conditioning length is fixed: truncate or right-pad (reference README.md:389, 512 tokens)."""
        return (ids + [self.pad_id] * length)[:length]

    def apply_chat_template(self, messages: List[dict], add_generation_prompt: bool = True,
                            n_vision_tokens: Sequence[int] = ()) -> List[int]:
        """messages: [{'role', 'content'}], content a string or a list of parts with 'type' in
        {'text', 'image_url', 'video_url'}; each media part expands to vision_start + pads + vision_end.
        `n_vision_tokens` has one entry per media part, in order: the number of (merged) vision tokens, or for a
        clip `{"per_frame": tokens per temporal group, "timestamps": [seconds of every group]}` (see `video_layout`)."""
        ids: List[int] = []
        vis = list(n_vision_tokens)
        for m in messages:
            ids += self.encode(f"<|im_start|>{m['role']}\n")
            content = m["content"]
            if isinstance(content, str):
                ids += self.encode(content)
            else:
                for part in content:
                    kind = part.get("type")
                    if kind == "text":
                        ids += self.encode(part["text"])
                    elif kind in ("image_url", "video_url", "image", "video"):
                        n = vis.pop(0) if vis else 0
                        pad = self.image_pad_id if kind.startswith("image") else self.video_pad_id
                        v0, v1 = self.special_ids["<|vision_start|>"], self.special_ids["<|vision_end|>"]
                        if isinstance(n, dict):
                            # a clip: one vision segment per temporal group, each after its time stamp
                            # ("<1.5 seconds>"), which is how Qwen3-VL lays videos out
                            for ts in n["timestamps"]:
                                ids += self.encode(f"<{ts:.1f} seconds>") + [v0] + [pad] * int(n["per_frame"]) + [v1]
                        else:
                            ids += [v0] + [pad] * n + [v1]
                    else:
                        raise ValueError(f"unknown content part type {kind!r}")
            ids += self.encode("<|im_end|>\n")
        if add_generation_prompt:
            ids += self.encode("<|im_start|>assistant\n")
        return ids


def video_layout(grid, frame_times: Sequence[float], temporal_patch: int = 2) -> dict:
    """Layout entry of a clip for `apply_chat_template`: grid (t, h, w) of merged vision tokens and the time
    (seconds) of every sampled frame -> tokens per temporal group and the group time stamps (mean of the first and
    last frame of each group; a trailing odd frame counts twice, as the vision encoder repeats it)."""
    t, h, w = grid
    times = list(frame_times)
    if len(times) % temporal_patch:
        times += [times[-1]] * (temporal_patch - len(times) % temporal_patch)
    stamps = [(times[i] + times[i + temporal_patch - 1]) / 2.0 for i in range(0, len(times), temporal_patch)][:t]
    return {"per_frame": h * w, "timestamps": stamps}


class HFTokenizer:
    """A checkpoint's own tokenizer (`tokenizer.json` + config, loaded by `transformers.AutoTokenizer`) behind the
    interface the framework uses everywhere (`ByteTokenizer` above): `encode` / `decode`, the ids of the end and
    media-placeholder tokens, `pad_or_truncate`, and the Qwen-style chat layout with every media part expanded to
    `<|vision_start|>` + n placeholder tokens + `<|vision_end|>` (n = merged vision tokens of that image / clip)."""

    NEEDED = ("<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")

    def __init__(self, hf):
        self.hf = hf
        self.vocab_size = len(hf)
        unk = hf.unk_token_id
        ids = {t: hf.convert_tokens_to_ids(t) for t in self.NEEDED + ("<|endoftext|>",)}
        missing = [t for t in self.NEEDED if ids[t] is None or (unk is not None and ids[t] == unk)]
        if missing:
            raise ValueError(f"tokenizer lacks the special tokens {missing}")
        self.special_ids: Dict[str, int] = {k: int(v) for k, v in ids.items() if v is not None}
        self.eos_id = self.special_ids["<|im_end|>"]
        eot = self.special_ids.get("<|endoftext|>")
        self.eot_id = eot if eot is not None and eot != unk else int(hf.eos_token_id if hf.eos_token_id is not None else self.eos_id)
        self.pad_id = int(hf.pad_token_id) if hf.pad_token_id is not None else self.eot_id
        self.pad_token_id = self.pad_id
        self.image_pad_id = self.special_ids["<|image_pad|>"]
        self.video_pad_id = self.special_ids["<|video_pad|>"]

    def encode(self, text: str) -> List[int]:
        return list(self.hf.encode(text, add_special_tokens=False))

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        return self.hf.decode([int(t) for t in ids], skip_special_tokens=skip_special)

    def pad_or_truncate(self, ids: List[int], length: int) -> List[int]:
        return (list(ids) + [self.pad_id] * length)[:length]

    apply_chat_template = ByteTokenizer.apply_chat_template   # same layout, built from encode() and special_ids


def load_tokenizer(checkpoint_path: Optional[str], vocab_size: int):
    """The checkpoint's tokenizer when it ships one (looked for in the directory itself and in `tokenizer/`),
    else the byte-level stand-in."""
    if checkpoint_path and Path(checkpoint_path).is_dir():
        for d in (Path(checkpoint_path), Path(checkpoint_path) / "tokenizer"):
            if (d / "tokenizer.json").exists():
                from transformers import AutoTokenizer

                return HFTokenizer(AutoTokenizer.from_pretrained(str(d)))
    return ByteTokenizer(vocab_size)

"""Prompt upsampling: the Reasoner rewrites a short user prompt into the dense structured caption
(JSON with subjects, lighting, cinematography, actions, ...) that the Generator was trained on.
Sampling settings follow the reference (README.md:131-141): max_tokens 20000, temperature 0.7,
top_p 0.8, top_k 20, presence_penalty 1.5, seed 3407."""
from __future__ import annotations

import json
from typing import Optional

from ..config import DecodingConfig

UPSAMPLER_DECODING = DecodingConfig(max_new_tokens=20000, do_sample=True, temperature=0.7, top_p=0.8, top_k=20,
                                    repetition_penalty=1.0, presence_penalty=1.5, seed=3407)
TOP_LEVEL_KEYS = ("subjects", "background_setting", "lighting", "aesthetics", "cinematography", "style_medium",
                  "artistic_style", "context", "actions", "text_and_signage_elements", "segments", "transitions",
                  "temporal_caption", "audio_description", "resolution", "aspect_ratio", "duration", "fps")
SYSTEM_PROMPT = ("Rewrite the user's request as one JSON object describing the video to generate, with the keys "
                 + ", ".join(TOP_LEVEL_KEYS) + ". Answer with the JSON object only.")


def upsample_prompt(reasoner, tokenizer, prompt: str, width: int, height: int, duration_s: float, fps: int,
                    decoding: Optional[DecodingConfig] = None) -> str:
    """Returns a compact JSON string; falls back to wrapping the raw prompt when the model's answer
    is not valid JSON (always the case with random-init weights)."""
    dc = decoding or UPSAMPLER_DECODING
    ids = tokenizer.apply_chat_template([{"role": "system", "content": SYSTEM_PROMPT},
                                         {"role": "user", "content": prompt}], True)
    out_ids, _ = reasoner.generate(ids, dc, (tokenizer.eos_id, tokenizer.eot_id))
    text = tokenizer.decode(out_ids)
    try:
        obj = json.loads(text[text.index("{"):text.rindex("}") + 1])
        if not isinstance(obj, dict):
            raise ValueError
    except ValueError:
        obj = {"temporal_caption": prompt}
    obj.setdefault("resolution", {"W": width, "H": height})
    obj.setdefault("duration", duration_s)
    obj.setdefault("fps", fps)
    return json.dumps(obj, separators=(",", ":"), ensure_ascii=False)


def main(argv=None) -> int:
    """`python -m cosmos_b200.utils.prompt_upsampler "a robot stacks blocks" --resolution 720 --num-frames 121 --fps 24`
    prints the dense caption (compact JSON) for the Generator and, on stderr, what the schema check found."""
    import argparse
    import sys

    import torch

    from ..config import resolve_size
    from ..io.prompt_schema import parse_prompt, validate_prompt
    from ..models.reasoner import ReasonerEngine
    from ..pipeline import Cosmos3OmniPipeline

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("prompt")
    ap.add_argument("--checkpoint-path", default="Cosmos3-Nano")
    ap.add_argument("--resolution", default="720")
    ap.add_argument("--aspect-ratio", default="16,9")
    ap.add_argument("--num-frames", type=int, default=189)
    ap.add_argument("--fps", type=int, default=24)
    ap.add_argument("--max-tokens", type=int, default=UPSAMPLER_DECODING.max_new_tokens)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    cuda = a.device.startswith("cuda")
    pipe = Cosmos3OmniPipeline.from_pretrained(a.checkpoint_path, torch_dtype=torch.bfloat16 if cuda else torch.float32,
                                               device_map=a.device if cuda else None, towers=("ar",),
                                               enable_safety_checker=False)
    w, h = resolve_size(a.resolution, a.aspect_ratio)
    import dataclasses
    dc = dataclasses.replace(UPSAMPLER_DECODING, max_new_tokens=a.max_tokens)
    text = upsample_prompt(ReasonerEngine(pipe.transformer, None), pipe.tokenizer, a.prompt, w, h, a.num_frames / a.fps, a.fps, dc)
    print(text)
    for problem in validate_prompt(parse_prompt(text) or {}):
        print(f"schema: {problem}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

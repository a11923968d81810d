"""Schema of the dense structured captions ("upsampled prompts") that the Generator is prompted with, and the
metadata rules for negative prompts.

A prompt file is one JSON object that is handed to the model as a compact JSON string (reference
cookbooks/cosmos3/generator/audiovisual/README.md:27-31). Its keys, read off the reference's prompt assets
(cookbooks/cosmos3/generator/audiovisual/assets/prompts/*/*.json, .../negative_prompts/*/neg_prompt.json,
cookbooks/cosmos3/generator/transfer/assets/*/prompt.json):

* `subjects[]` with 18 fields each, `background_setting`, `lighting{4}`, `aesthetics{4}`, `cinematography{6}`,
  `style_medium`, `artistic_style`, `context`, `actions[{time, description}]`, `text_and_signage_elements[]`,
  `segments[]`, `transitions[]`, `temporal_caption`, `audio_description`;
* metadata: `resolution{W, H}`, `aspect_ratio` ("16,9"), `duration` ("7s"), `fps`;
* text-to-image prompts add `subject_details`, `quadrant_scan`, `comprehensive_t2i_caption` (and subjects carry
  `number_of_hands` / `number_of_fingers` instead of `action` / `state_changes`);
* negative prompts add `physical_realism`.

Negative-prompt metadata (`negative_metadata_mode`, `negative_prompt_keep_metadata` of the input spec, reference
evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb:467-469,513-515): with `keep_metadata` false the
metadata keys a negative prompt file carries are dropped; mode "same" then gives the negative prompt the
positive prompt's metadata, mode "none" leaves it without."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

SUBJECT_FIELDS = ("description", "appearance_details", "relationship", "location", "relative_size", "orientation",
                  "pose", "action", "state_changes", "clothing", "expression", "gender", "age",
                  "skin_tone_and_texture", "facial_features", "number_of_subjects", "number_of_arms", "number_of_legs")
SUBJECT_FIELDS_T2I = ("number_of_hands", "number_of_fingers")
NESTED_FIELDS = {
    "lighting": ("conditions", "direction", "shadows", "illumination_effect"),
    "aesthetics": ("composition", "color_scheme", "mood_atmosphere", "patterns"),
    "cinematography": ("camera_motion", "framing", "camera_angle", "depth_of_field", "focus", "lens_focal_length"),
    "quadrant_scan": ("top_left", "top_right", "bottom_left", "bottom_right", "absolute_center"),
    "resolution": ("W", "H"),
}
LIST_ITEM_FIELDS = {
    "actions": ("time", "description"),
    "segments": ("segment_index", "time_range", "description", "key_changes", "camera"),
    "text_and_signage_elements": ("text", "category", "appearance", "spatial_temporal", "context"),
}
STRING_KEYS = ("background_setting", "style_medium", "artistic_style", "context", "temporal_caption",
               "audio_description", "comprehensive_t2i_caption", "physical_realism", "aspect_ratio", "duration")
METADATA_KEYS = ("resolution", "aspect_ratio", "duration", "fps")
TOP_LEVEL_KEYS = (("subjects", "subject_details") + tuple(NESTED_FIELDS) + tuple(LIST_ITEM_FIELDS) + ("transitions",)
                  + STRING_KEYS + ("fps",))


def parse_prompt(text: str) -> Optional[Dict[str, Any]]:
    """The JSON object of a structured prompt, or None for a plain-text prompt."""
    t = text.strip()
    if not t.startswith("{"):
        return None
    try:
        obj = json.loads(t)
    except json.JSONDecodeError:
        return None
    return obj if isinstance(obj, dict) else None


def compact(obj: Dict[str, Any]) -> str:
    return json.dumps(obj, separators=(",", ":"), ensure_ascii=False)


def validate_prompt(obj: Dict[str, Any]) -> List[str]:
    """Problems of a structured prompt as a list of messages (empty = conforms). Unknown keys are reported,
    not rejected: the model reads the string either way."""
    bad: List[str] = []
    for k, v in obj.items():
        if k not in TOP_LEVEL_KEYS:
            bad.append(f"unknown key '{k}'")
        elif k in STRING_KEYS and not isinstance(v, str):
            bad.append(f"'{k}' must be a string")
        elif k == "fps" and not isinstance(v, (int, float)):
            bad.append("'fps' must be a number")
        elif k in NESTED_FIELDS:
            if not isinstance(v, dict):
                bad.append(f"'{k}' must be an object")
            else:
                bad += [f"unknown key '{k}.{f}'" for f in v if f not in NESTED_FIELDS[k]]
        elif k in LIST_ITEM_FIELDS or k in ("subjects", "transitions"):
            if not isinstance(v, list):
                bad.append(f"'{k}' must be a list")
                continue
            allowed = SUBJECT_FIELDS + SUBJECT_FIELDS_T2I if k == "subjects" else LIST_ITEM_FIELDS.get(k)
            for i, item in enumerate(v):
                if allowed is None:
                    continue
                if not isinstance(item, dict):
                    bad.append(f"'{k}[{i}]' must be an object")
                else:
                    bad += [f"unknown key '{k}[{i}].{f}'" for f in item if f not in allowed]
        elif k == "subject_details" and not isinstance(v, dict):
            bad.append("'subject_details' must be an object")
    res = obj.get("resolution")
    if isinstance(res, dict) and not all(isinstance(res.get(a), int) and res.get(a) > 0 for a in ("W", "H")):
        bad.append("'resolution' needs positive integers W and H")
    return bad


def make_metadata(width: int, height: int, num_frames: int, fps: int, aspect_ratio: Optional[str] = None) -> Dict[str, Any]:
    """Metadata block in the reference's spelling: {"resolution": {"W", "H"}, "aspect_ratio": "16,9",
    "duration": "7s", "fps": 24}; images (one frame) carry no duration or fps."""
    from math import gcd
    if aspect_ratio is None:
        g = gcd(width, height) or 1
        aspect_ratio = f"{width // g},{height // g}"
    meta: Dict[str, Any] = {"resolution": {"W": int(width), "H": int(height)}, "aspect_ratio": aspect_ratio}
    if num_frames > 1:
        meta["duration"] = f"{max(1, round(num_frames / float(fps)))}s"
        meta["fps"] = int(fps)
    return meta


def metadata_of(obj: Dict[str, Any]) -> Dict[str, Any]:
    return {k: obj[k] for k in METADATA_KEYS if k in obj}


def negative_prompt_for(negative: str, positive: str, mode: str = "none", keep_metadata: bool = False,
                        fallback_metadata: Optional[Dict[str, Any]] = None) -> str:
    """Applies `negative_metadata_mode` / `negative_prompt_keep_metadata` to a negative prompt.

    Structured (JSON) negative prompts lose their own metadata keys unless `keep_metadata`; mode "same" then
    copies the positive prompt's metadata (or `fallback_metadata` when the positive prompt is plain text or has
    none) for every key the negative prompt does not keep. Plain-text negative prompts pass through: their
    metadata is the resolution / duration sentence that the pipeline appends (`negative_metadata_same`)."""
    if mode not in ("none", "same"):
        raise ValueError("negative_metadata_mode must be 'none' or 'same'")
    obj = parse_prompt(negative)
    if obj is None:
        return negative
    if not keep_metadata:
        obj = {k: v for k, v in obj.items() if k not in METADATA_KEYS}
    if mode == "same":
        pos = parse_prompt(positive)
        src = metadata_of(pos) if pos else {}
        if not src and fallback_metadata:
            src = fallback_metadata
        for k in METADATA_KEYS:
            if k in src and k not in obj:
                obj[k] = src[k]
    return compact(obj)

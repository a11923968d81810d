"""Prompting conventions of the Reasoner: sampling presets, the reasoning toggle, message layout, the
0-1000 coordinate convention for boxes / points / trajectories, and parsers for the JSON answers.

Follows the reference's prompt guide (cookbooks/cosmos3/reasoner/reasoner_prompt_guide.md): sampling
parameters with and without reasoning (:7-27), system prompt (:35-39), reasoning switched on by a suffix of
the user prompt (:41-57), media parts before the text part (:59-75), boxes `[x1, y1, x2, y2]` and points
`[x, y]` normalised to 0-1000 per axis with the origin at the top left (:77-99), event lists with `start`,
`end`, `caption` and times in seconds or `mm:ss.ff` (:160, :222)."""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

from ..config import DecodingConfig

SYSTEM_PROMPT = "You are a helpful assistant."
DECODING_DIRECT = DecodingConfig(do_sample=True, temperature=0.7, top_p=0.8, top_k=20, repetition_penalty=1.0,
                                 presence_penalty=1.5)
DECODING_REASONING = DecodingConfig(do_sample=True, temperature=0.6, top_p=0.95, top_k=20, repetition_penalty=1.0,
                                    presence_penalty=0.0)
VIDEO_PROCESSOR_KWARGS = {"fps": 4, "do_sample_frames": True}   # `extra_body.mm_processor_kwargs` for video inputs
REASONING_SUFFIX = ("Answer the question using the following format:\n\n<think>\nYour reasoning.\n</think>\n\n"
                    "Write your final answer immediately after the </think> tag.")
COORD_RANGE = 1000


def with_reasoning(prompt: str) -> str:
    """Reasoning is requested through the user prompt: the format instruction goes after the task text."""
    return prompt.rstrip() + "\n\n" + REASONING_SUFFIX


def decoding_for(reasoning: bool, **overrides) -> DecodingConfig:
    base = DECODING_REASONING if reasoning else DECODING_DIRECT
    return DecodingConfig(**{**base.__dict__, **overrides})


def build_messages(text: str, images: Sequence[str] = (), videos: Sequence[str] = (), system: Optional[str] = SYSTEM_PROMPT,
                   reasoning: bool = False) -> List[Dict[str, Any]]:
    """OpenAI-style chat messages with every media part before the text part."""
    content: List[Dict[str, Any]] = [{"type": "image_url", "image_url": {"url": u}} for u in images]
    content += [{"type": "video_url", "video_url": {"url": u}} for u in videos]
    content.append({"type": "text", "text": with_reasoning(text) if reasoning else text})
    msgs: List[Dict[str, Any]] = [{"role": "system", "content": system}] if system else []
    msgs.append({"role": "user", "content": content})
    return msgs


def split_reasoning(answer: str) -> Tuple[str, str]:
    """(reasoning, final answer) of a completion; reasoning is '' when the model did not think aloud.
    An unterminated <think> block (generation cut off) counts entirely as reasoning."""
    m = re.search(r"<think>(.*?)</think>", answer, flags=re.S)
    if m:
        return m.group(1).strip(), answer[m.end():].strip()
    if "<think>" in answer:
        return answer.split("<think>", 1)[1].strip(), ""
    if "</think>" in answer:      # chat templates may open the block themselves
        head, tail = answer.split("</think>", 1)
        return head.strip(), tail.strip()
    return "", answer.strip()


# ------------------------------------------------------------------ coordinates
def to_normalized(xy: Sequence[float], width: int, height: int) -> List[int]:
    """Pixel coordinates (x, y, [x2, y2, ...]) -> 0-1000, each axis on its own scale."""
    return [int(round(min(max(v / (width if i % 2 == 0 else height), 0.0), 1.0) * COORD_RANGE)) for i, v in enumerate(xy)]


def from_normalized(xy: Sequence[float], width: int, height: int) -> List[float]:
    return [float(v) / COORD_RANGE * (width if i % 2 == 0 else height) for i, v in enumerate(xy)]


# ------------------------------------------------------------------ answers
def parse_json_answer(answer: str) -> Any:
    """The JSON value in a completion: fenced ```json blocks first, else the first [...] or {...} span that
    parses; the reasoning block is ignored. Raises ValueError when there is none."""
    _, final = split_reasoning(answer)
    text = final or answer
    for block in re.findall(r"```(?:json)?\s*(.*?)```", text, flags=re.S):
        try:
            return json.loads(block)
        except json.JSONDecodeError:
            continue
    pairs = sorted((("[", "]"), ("{", "}")), key=lambda oc: text.find(oc[0]) if oc[0] in text else len(text))
    for open_c, close_c in pairs:      # the opener that comes first is the outer value
        start = text.find(open_c)
        while start >= 0:
            end = text.rfind(close_c)
            while end > start:
                try:
                    return json.loads(text[start:end + 1])
                except json.JSONDecodeError:
                    end = text.rfind(close_c, start, end)
            start = text.find(open_c, start + 1)
    raise ValueError("no JSON value in the answer")


def _items(answer: str) -> List[Dict[str, Any]]:
    v = parse_json_answer(answer)
    if isinstance(v, dict):
        v = [v]
    return [it for it in v if isinstance(it, dict)] if isinstance(v, list) else []


def parse_boxes(answer: str, width: Optional[int] = None, height: Optional[int] = None) -> List[Dict[str, Any]]:
    """[{'bbox_2d': [x1, y1, x2, y2], 'label': ...}]; with an image size the boxes come back in pixels."""
    out = []
    for it in _items(answer):
        b = it.get("bbox_2d")
        if isinstance(b, list) and len(b) == 4 and all(isinstance(v, (int, float)) for v in b):
            box = from_normalized(b, width, height) if width and height else [float(v) for v in b]
            out.append({"bbox_2d": box, "label": it.get("label", "")})
    return out


def parse_points(answer: str, width: Optional[int] = None, height: Optional[int] = None) -> List[Dict[str, Any]]:
    """[{'point_2d': [x, y], 'label': ...}] in answer order (a trajectory is the list of its points)."""
    out = []
    for it in _items(answer):
        p = it.get("point_2d")
        if isinstance(p, list) and len(p) == 2 and all(isinstance(v, (int, float)) for v in p):
            pt = from_normalized(p, width, height) if width and height else [float(v) for v in p]
            out.append({"point_2d": pt, "label": it.get("label", "")})
    return out


def parse_timestamp(t) -> float:
    """Seconds from a number, 'ss.ff', 'mm:ss.ff' or 'hh:mm:ss.ff'."""
    if isinstance(t, (int, float)):
        return float(t)
    parts = str(t).strip().rstrip("s").split(":")
    if not 1 <= len(parts) <= 3:
        raise ValueError(f"bad timestamp {t!r}")
    sec = 0.0
    for p in parts:
        sec = sec * 60.0 + float(p)
    return sec


def format_timestamp(seconds: float) -> str:
    """'mm:ss.ff' (hundredths)."""
    cs = int(round(max(seconds, 0.0) * 100))
    return f"{cs // 6000:02d}:{(cs // 100) % 60:02d}.{cs % 100:02d}"


def parse_events(answer: str) -> List[Dict[str, Any]]:
    """[{'start': s, 'end': s, 'caption': ...}] with times in seconds, whatever format the answer used."""
    out = []
    for it in _items(answer):
        if "start" in it and "end" in it:
            out.append({"start": parse_timestamp(it["start"]), "end": parse_timestamp(it["end"]),
                        "caption": it.get("caption", "")})
    return out


# ------------------------------------------------------------------ task prompts
def grounding_prompt(target: str) -> str:
    return (f"Locate {target} in the image. Return a json list of objects with the keys \"bbox_2d\" "
            "([x1, y1, x2, y2], normalized 0-1000) and \"label\".")


def trajectory_prompt(task: str, label: str = "gripper trajectory") -> str:
    return (f"You are given the task \"{task}\". Specify the 2D trajectory your end effector should follow. Return the "
            f"trajectory coordinates in JSON format like this: {{\"point_2d\": [x, y], \"label\": \"{label}\"}}.")


def events_prompt(time_format: str = "seconds") -> str:
    if time_format not in ("seconds", "mm:ss.ff"):
        raise ValueError("time_format must be 'seconds' or 'mm:ss.ff'")
    return ("Describe the notable events in the provided video. Provide the result in json format with "
            f"'{time_format}' for time depiction for each event. Use keywords 'start', 'end' and 'caption' in the json output.")

"""Per-sample input specs of the inference CLI: JSON (one sample) or JSONL (one per line).

The key set, defaults and validation rules follow the reference's cookbooks: key list and
modes in cookbooks/cosmos3/generator/audiovisual/run_with_cosmos_framework.ipynb:303-422,
action/run_fd_with_cosmos_framework.ipynb:475-488, action/run_id_with_cosmos_framework.ipynb:450-462,
transfer/specs/*.json, evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb:460-523 and
reasoner/README.md:22-29. Validation is strict: unknown keys and invalid combinations raise
(the reference notes that `enable_sound` must be false for the reasoner to pass validation,
reasoner/README.md:22-23). Relative paths are resolved against the spec file's directory.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

MODEL_MODES = ("text2image", "text2video", "image2video", "video2video", "forward_dynamics",
               "inverse_dynamics", "policy", "reasoner")
CONTROL_KEYS = ("edge", "blur", "depth", "seg", "wsm")
DOMAINS = ("av", "droid_lerobot", "umi", "bridge_orig_lerobot", "camera_pose")
FPS_CHOICES = (10, 15, 16, 20, 24, 30)
PATH_KEYS = ("prompt_path", "negative_prompt_file", "vision_path", "action_path")


class SpecError(ValueError):
    pass


@dataclass
class InferenceSpec:
    model_mode: str = "text2video"
    name: str = "sample"
    prompt: Optional[str] = None
    prompt_path: Optional[str] = None
    negative_prompt: Optional[str] = None
    negative_prompt_file: Optional[str] = None
    negative_metadata_mode: str = "none"
    negative_prompt_keep_metadata: bool = False
    enable_sound: bool = False
    num_steps: int = 35
    guidance: float = 6.0
    control_guidance: Optional[float] = None
    guidance_interval: Sequence[float] = (0, 1000)
    normalize_cfg: bool = False
    shift: float = 10.0
    sigma_max: Optional[float] = None
    fps: int = 24
    num_frames: int = 189
    resolution: str = "720"
    aspect_ratio: str = "16,9"
    seed: int = 0
    num_outputs: int = 1
    vision_path: Optional[str] = None
    condition_frame_indexes_vision: Optional[List[int]] = None
    num_video_frames_per_chunk: Optional[int] = None
    num_conditional_frames: Optional[int] = None
    num_first_chunk_conditional_frames: Optional[int] = None
    share_vision_temporal_positions: bool = False
    edge: Optional[Dict[str, Any]] = None
    blur: Optional[Dict[str, Any]] = None
    depth: Optional[Dict[str, Any]] = None
    seg: Optional[Dict[str, Any]] = None
    wsm: Optional[Dict[str, Any]] = None
    action_chunk_size: Optional[int] = None
    action_path: Optional[str] = None
    raw_action_dim: Optional[int] = None
    domain_name: Optional[str] = None
    image_size: Optional[int] = None
    view_point: Optional[str] = None
    max_new_tokens: int = 4096
    do_sample: bool = True
    temperature: float = 0.7
    top_p: float = 0.8
    top_k: int = 20
    repetition_penalty: float = 1.0
    presence_penalty: float = 1.5
    scheduler: str = "euler"
    # filled by the loader
    spec_dir: Optional[str] = None

    # ------------------------------------------------------------------ derived
    @property
    def controls(self) -> Dict[str, Dict[str, Any]]:
        return {k: getattr(self, k) for k in CONTROL_KEYS if getattr(self, k) is not None}

    @property
    def is_transfer(self) -> bool:
        """Presence of any control hint key selects transfer inference (transfer/README.md:35)."""
        return bool(self.controls)

    @property
    def is_generator(self) -> bool:
        return self.model_mode != "reasoner"

    def resolve(self, p: Optional[str]) -> Optional[Path]:
        if p is None:
            return None
        path = Path(p)
        if not path.is_absolute() and self.spec_dir:
            path = Path(self.spec_dir) / path
        return path

    def prompt_text(self) -> str:
        if self.prompt is not None:
            return self.prompt
        if self.prompt_path is not None:
            return _read_prompt_file(self.resolve(self.prompt_path))
        return ""

    def negative_prompt_text(self, size: Optional[Tuple[int, int]] = None) -> str:
        """The negative prompt after `negative_metadata_mode` / `negative_prompt_keep_metadata` (see
        io/prompt_schema.py); `size` = (width, height) supplies the metadata when the positive prompt has none."""
        from .prompt_schema import make_metadata, negative_prompt_for
        if self.negative_prompt is not None:
            neg = self.negative_prompt
        elif self.negative_prompt_file is not None:
            neg = _read_prompt_file(self.resolve(self.negative_prompt_file))
        else:
            return ""
        fallback = None
        if size is not None:
            fallback = make_metadata(size[0], size[1], self.num_frames, self.fps,
                                     self.aspect_ratio)
        return negative_prompt_for(neg, self.prompt_text(), self.negative_metadata_mode,
                                   self.negative_prompt_keep_metadata, fallback)

    def to_dict(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self) if f.name != "spec_dir"}


def _read_prompt_file(path: Path) -> str:
    """Prompt files are JSON documents (dense structured captions); they are fed to the model as
    a compact JSON string (audiovisual/README.md:27-31). Plain-text files are passed through."""
    text = Path(path).read_text()
    try:
        return json.dumps(json.loads(text), separators=(",", ":"), ensure_ascii=False)
    except json.JSONDecodeError:
        return text.strip()


_FIELD_NAMES = {f.name for f in fields(InferenceSpec)} - {"spec_dir"}


def _type_check(d: Dict[str, Any]) -> None:
    def need(key, types, allow_none=False):
        if key in d and not (isinstance(d[key], types) or (allow_none and d[key] is None)):
            raise SpecError(f"'{key}' must be {types}, got {type(d[key]).__name__}")

    for k in ("name", "model_mode", "resolution", "aspect_ratio"):
        need(k, str)
    for k in ("prompt", "prompt_path", "negative_prompt", "negative_prompt_file", "vision_path", "action_path",
              "domain_name", "view_point"):
        need(k, str, True)
    for k in ("num_steps", "fps", "num_frames", "seed", "num_outputs", "max_new_tokens", "top_k"):
        if k in d and (isinstance(d[k], bool) or not isinstance(d[k], int)):
            raise SpecError(f"'{k}' must be an integer")
    for k in ("guidance", "shift", "temperature", "top_p", "repetition_penalty", "presence_penalty"):
        if k in d and (isinstance(d[k], bool) or not isinstance(d[k], (int, float))):
            raise SpecError(f"'{k}' must be a number")
    for k in ("enable_sound", "normalize_cfg", "negative_prompt_keep_metadata", "share_vision_temporal_positions",
              "do_sample"):
        need(k, bool)


def validate(spec: InferenceSpec) -> InferenceSpec:
    s = spec
    if s.model_mode not in MODEL_MODES:
        raise SpecError(f"model_mode must be one of {MODEL_MODES}, got {s.model_mode!r}")
    if not s.name or "/" in s.name or s.name in (".", ".."):
        raise SpecError("name must be a non-empty directory name")
    if s.prompt is not None and s.prompt_path is not None:
        raise SpecError("give either prompt or prompt_path, not both")
    if s.negative_prompt is not None and s.negative_prompt_file is not None:
        raise SpecError("give either negative_prompt or negative_prompt_file, not both")
    if s.negative_metadata_mode not in ("none", "same"):
        raise SpecError("negative_metadata_mode must be 'none' or 'same'")
    if s.model_mode == "reasoner":
        if s.enable_sound:
            raise SpecError("enable_sound must be false for model_mode 'reasoner'")
        if s.is_transfer:
            raise SpecError("control hints are not valid for model_mode 'reasoner'")
        if s.max_new_tokens < 1:
            raise SpecError("max_new_tokens must be >= 1")
        if not (0.0 < s.top_p <= 1.0) or s.top_k < 0 or s.temperature < 0 or s.repetition_penalty <= 0:
            raise SpecError("invalid decoding parameters")
        return s
    # generator modes
    from ..config import ASPECT_RATIOS, RESOLUTIONS_16_9
    if str(s.resolution) not in RESOLUTIONS_16_9:
        raise SpecError(f"resolution must be one of {sorted(RESOLUTIONS_16_9)}")
    if s.aspect_ratio not in ASPECT_RATIOS:
        raise SpecError(f"aspect_ratio must be one of {ASPECT_RATIOS}")
    if s.fps not in FPS_CHOICES:
        raise SpecError(f"fps must be one of {FPS_CHOICES}")
    if not (1 <= s.num_frames <= 300):
        raise SpecError("num_frames must be in [1, 300]")
    if s.num_frames != 1 and (s.num_frames - 1) % 4 != 0:
        raise SpecError("num_frames must be 1 or 1 + 4k (the tokenizer compresses time 4x after the first frame)")
    if s.num_steps < 1 or s.num_outputs < 1:
        raise SpecError("num_steps and num_outputs must be >= 1")
    if s.shift <= 0 or (s.sigma_max is not None and s.sigma_max <= 0):
        raise SpecError("shift and sigma_max must be positive")
    gi = list(s.guidance_interval)
    if len(gi) != 2 or gi[0] > gi[1]:
        raise SpecError("guidance_interval must be [lo, hi] with lo <= hi")
    if s.scheduler not in ("euler", "unipc"):
        raise SpecError("scheduler must be 'euler' or 'unipc'")
    if s.model_mode == "text2image" and s.num_frames != 1:
        raise SpecError("text2image needs num_frames == 1")
    if s.model_mode == "text2image" and s.enable_sound:
        raise SpecError("enable_sound is not valid for text2image")
    if s.model_mode in ("image2video", "video2video", "forward_dynamics", "inverse_dynamics", "policy") \
            and s.vision_path is None and not s.is_transfer:
        raise SpecError(f"model_mode '{s.model_mode}' needs vision_path")
    if s.model_mode in ("text2image", "text2video") and s.vision_path is not None:
        raise SpecError(f"vision_path is not valid for model_mode '{s.model_mode}'")
    if s.is_transfer:
        if s.model_mode != "video2video":
            raise SpecError("control hints need model_mode 'video2video'")
        if s.num_outputs != 1:
            raise SpecError("transfer inference needs batch size 1 (num_outputs == 1)")
        for k, v in s.controls.items():
            if not isinstance(v, dict) or "control_path" not in v:
                raise SpecError(f"'{k}' must be an object with 'control_path'")
            extra = set(v) - {"control_path", "preset_edge_threshold", "preset_blur_strength", "control_weight"}
            if extra:
                raise SpecError(f"unknown keys in '{k}': {sorted(extra)}")
    elif s.control_guidance is not None:
        raise SpecError("control_guidance needs a control hint (edge/blur/depth/seg/wsm)")
    if s.model_mode in ("forward_dynamics", "inverse_dynamics", "policy"):
        if s.domain_name not in DOMAINS:
            raise SpecError(f"domain_name must be one of {DOMAINS}")
        if not s.action_chunk_size or s.action_chunk_size < 1:
            raise SpecError("action modes need action_chunk_size >= 1")
        if s.model_mode == "forward_dynamics" and s.action_path is None:
            raise SpecError("forward_dynamics needs action_path")
        if s.image_size is not None and s.image_size not in (256, 480, 720):
            raise SpecError("image_size must be 256, 480 or 720")
    else:
        for k in ("action_chunk_size", "action_path", "domain_name"):
            if getattr(s, k) is not None:
                raise SpecError(f"'{k}' is only valid for action modes")
    if s.condition_frame_indexes_vision is not None:
        idx = s.condition_frame_indexes_vision
        t_lat = (s.num_frames - 1) // 4 + 1
        if any((not isinstance(i, int)) or i < 0 or i >= t_lat for i in idx):
            raise SpecError(f"condition_frame_indexes_vision must index latent frames in [0, {t_lat})")
    return s


def spec_from_dict(d: Dict[str, Any], spec_dir: Optional[Union[str, Path]] = None,
                   overrides: Optional[Dict[str, Any]] = None) -> InferenceSpec:
    if not isinstance(d, dict):
        raise SpecError("a sample spec must be a JSON object")
    unknown = set(d) - _FIELD_NAMES
    if unknown:
        raise SpecError(f"unknown spec keys: {sorted(unknown)}")
    _type_check(d)
    d = dict(d)
    mode = d.get("model_mode", "text2video")
    # mode-dependent defaults (recipes of the reference's cookbooks)
    if mode == "text2image":
        d.setdefault("num_frames", 1)
    if mode in ("forward_dynamics", "inverse_dynamics", "policy"):
        d.setdefault("guidance", 1.0)
        d.setdefault("num_steps", 30)
        if "action_chunk_size" in d and isinstance(d["action_chunk_size"], int):
            d.setdefault("num_frames", d["action_chunk_size"] + 1)
        d.setdefault("fps", {"av": 10, "droid_lerobot": 15, "umi": 20}.get(d.get("domain_name"), 10))
    if overrides:
        d.update({k: v for k, v in overrides.items() if v is not None})
    if "resolution" in d:
        d["resolution"] = str(d["resolution"])
    spec = InferenceSpec(**d)
    spec.spec_dir = None if spec_dir is None else str(spec_dir)
    if mode in ("forward_dynamics", "inverse_dynamics", "policy") and spec.image_size is not None \
            and "resolution" not in d:
        spec.resolution = str(spec.image_size)
    return validate(spec)


def load_specs(path: Union[str, Path], overrides: Optional[Dict[str, Any]] = None) -> List[InferenceSpec]:
    """`.json` = one sample, `.jsonl` = one sample per non-empty line."""
    path = Path(path)
    if not path.exists():
        raise SpecError(f"spec file not found: {path}")
    text = path.read_text()
    base = path.resolve().parent
    try:
        if path.suffix == ".jsonl":
            rows = []
            for n, line in enumerate(text.splitlines(), 1):
                if not line.strip():
                    continue
                try:
                    rows.append(json.loads(line))
                except json.JSONDecodeError as e:
                    raise SpecError(f"{path}:{n}: invalid JSON ({e})") from e
        else:
            doc = json.loads(text)
            rows = doc if isinstance(doc, list) else [doc]
    except json.JSONDecodeError as e:
        raise SpecError(f"{path}: invalid JSON ({e})") from e
    if not rows:
        raise SpecError(f"{path}: no samples")
    specs = [spec_from_dict(r, base, overrides) for r in rows]
    names = [s.name for s in specs]
    if len(set(names)) != len(names):
        raise SpecError("sample names must be unique within a spec file (they name output directories)")
    return specs

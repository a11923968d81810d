"""Hugging Face front end for the Reasoner: `Cosmos3ReasonerForConditionalGeneration` with the usual
`from_pretrained` / `generate` calls, registered with the `transformers` auto classes under the model
type `cosmos3_reasoner` (what the reference's `packages/transformers-cosmos3` and `packages/vllm-cosmos3`
plug-ins provide for its checkpoints: reference cookbooks/cosmos3/reasoner/run_with_vllm.ipynb:132-133,
cookbooks/cosmos3/README.md:165-166). The model underneath is this package's AR tower + vision encoder;
generation runs through `ReasonerEngine` (contiguous KV) and follows the decoding defaults of
`DecodingConfig`.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .config import DecodingConfig, MoTConfig, get_model_config
from .models.mot import MoTModel
from .models.reasoner import ReasonerEngine
from .models.vit import VisionEncoder

try:  # transformers is optional: without it the class below is a plain nn.Module with the same methods
    from transformers import AutoConfig, AutoModelForCausalLM, PretrainedConfig, PreTrainedModel
    _HAVE_HF = True
except Exception:  # noqa: BLE001 - any import problem means "no transformers"
    PretrainedConfig, PreTrainedModel = object, torch.nn.Module
    _HAVE_HF = False


class Cosmos3ReasonerConfig(PretrainedConfig):
    model_type = "cosmos3_reasoner"

    def __init__(self, arch: str = "Cosmos3-Nano", overrides: Optional[dict] = None, **kw):
        self.arch = arch
        self.overrides = dict(overrides or {})
        if _HAVE_HF:
            super().__init__(**kw)

    def mot_config(self) -> MoTConfig:
        return get_model_config(self.arch, **{k: tuple(v) if isinstance(v, list) else v for k, v in self.overrides.items()})


class Cosmos3ReasonerForConditionalGeneration(PreTrainedModel):
    config_class = Cosmos3ReasonerConfig
    base_model_prefix = "model"

    def __init__(self, config: Cosmos3ReasonerConfig, dtype=torch.float32, device="cpu"):
        if _HAVE_HF:
            super().__init__(config)
        else:
            super().__init__()
            self.config = config
        cfg = config.mot_config()
        self.model = MoTModel(cfg, dtype=dtype, device=device, towers=("ar",))
        self.visual = VisionEncoder(cfg).to(device=device, dtype=dtype)
        self.model.init_weights(seed=0)

    def _init_weights(self, module):  # weights come from init_weights / a checkpoint, not from HF's initialiser
        return

    @classmethod
    def from_pretrained(cls, name_or_path: str, torch_dtype=torch.float32, device_map: Optional[str] = None,
                        config_overrides: Optional[dict] = None, **_):
        """`name_or_path`: an architecture name (random-init weights) or a directory with `transformer/` safetensors
        in this package's checkpoint layout."""
        from pathlib import Path

        from .ckpt import safetensors_io as sio

        p = Path(name_or_path)
        arch = name_or_path
        if (p / "config.json").exists() and not (p / "transformer").exists():
            return cls.from_qwen3vl(p, torch_dtype, device_map)
        if (p / "transformer" / "config.json").exists():
            import json
            arch = json.loads((p / "transformer" / "config.json").read_text()).get("name", "Cosmos3-Nano")
        arch = arch.split("/")[-1]
        m = cls(Cosmos3ReasonerConfig(arch, config_overrides), dtype=torch_dtype, device=device_map or "cpu")
        if (p / "transformer").exists():
            state = {k: v for k, v in sio.model_state(m.model).items()}
            sio.load_into(p / "transformer", {k: v.data for k, v in state.items()}, strict=False)
        return m.eval()

    @classmethod
    def from_qwen3vl(cls, model_dir, torch_dtype=torch.float32, device_map: Optional[str] = None):
        """A checkpoint directory in the Hugging Face Qwen3-VL layout (`config.json` with `text_config` and
        `vision_config`, safetensors shards): the shapes come from its config, the tensors are mapped by
        ckpt/hf_qwen3vl.py. The Reasoner is Qwen3-VL-based, so this is how it starts from public weights."""
        import json
        from pathlib import Path
        from types import SimpleNamespace

        from .ckpt import hf_qwen3vl as hq

        doc = json.loads((Path(model_dir) / "config.json").read_text())
        if "text_config" not in doc:
            raise ValueError(f"{model_dir}/config.json has no text_config: not a Qwen3-VL checkpoint")
        text, vision = SimpleNamespace(**doc["text_config"]), doc.get("vision_config")
        text.rms_norm_eps = getattr(text, "rms_norm_eps", 1e-6)
        kw = hq.config_kwargs_from_hf(text, SimpleNamespace(**vision) if vision else None)
        kw = {k: (list(v) if isinstance(v, tuple) else v) for k, v in kw.items()}
        m = cls(Cosmos3ReasonerConfig("tiny", kw), dtype=torch_dtype, device=device_map or "cpu")
        hq.load_checkpoint_dir(m.model, m.visual if vision else None, model_dir)
        return m.eval()

    def save_qwen3vl(self, out_dir, token_ids: Optional[dict] = None) -> None:
        """Writes a checkpoint directory in the Hugging Face Qwen3-VL layout (`config.json` + safetensors with the
        text tower, LM head and vision tower) that `transformers` and engines built on it load as
        `Qwen3VLForConditionalGeneration`."""
        import json
        from pathlib import Path

        from .ckpt import hf_qwen3vl as hq
        from .ckpt import safetensors_io as sio
        state = hq.export_text_weights(self.model)
        state.update(hq.export_vision_weights(self.visual))
        sio.save_sharded(state, out_dir)
        (Path(out_dir) / "config.json").write_text(json.dumps(hq.hf_config_dict(self.model.cfg, token_ids), indent=1))

    def _encode_images(self, pixel_values: torch.Tensor, image_grid_thw: Optional[torch.Tensor]):
        """Vision rows, token grids and DeepStack features of the images of a prompt. `pixel_values`: [T, 3, H, W] in
        [-1, 1] (one image / clip) or the patch rows of a `transformers` Qwen3-VL processor with `image_grid_thw`."""
        vp = next(self.visual.parameters())
        vdt, vdev = vp.dtype, vp.device
        if pixel_values.dim() != 2:
            ve, grid, deep = self.visual(pixel_values.to(device=vdev, dtype=vdt), return_deepstack=True)
            return ve, [grid], deep
        from .ckpt.hf_qwen3vl import frames_from_hf_patches
        cfg = self.model.cfg
        if image_grid_thw is None:
            raise ValueError("pixel_values in patch-row layout need image_grid_thw")
        embs, grids, deeps, row = [], [], [], 0
        for g in image_grid_thw.tolist():
            n = int(g[0] * g[1] * g[2])
            frames = frames_from_hf_patches(pixel_values[row:row + n], g, cfg.vit_patch, cfg.vit_temporal_patch,
                                            cfg.vit_spatial_merge)
            row += n
            e, grid, d = self.visual(frames.to(device=vdev, dtype=vdt), return_deepstack=True)
            embs.append(e), grids.append(grid), deeps.append(d)
        deep = [torch.cat([d[k] for d in deeps]) for k in range(len(deeps[0]))] if deeps[0] else None
        return torch.cat(embs), grids, deep

    def forward(self, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor] = None,
                image_grid_thw: Optional[torch.Tensor] = None, image_token_id: Optional[int] = None, **_):
        """Teacher-forced logits [1, S, V] (no KV reuse); with `pixel_values` the positions that hold `image_token_id`
        take the vision rows, 3-D rotary ids and DeepStack features."""
        from .models import rope
        cfg = self.model.cfg
        ids = input_ids.clamp(max=cfg.vocab_size - 1)
        if pixel_values is None:
            x = self.model.embed_tokens(ids)
            h, _ = self.model.ar_forward(x, rope.text_positions(ids.shape[1], 0, ids.device))
            return self.model.lm_logits(h).float()
        if image_token_id is None:
            raise ValueError("image_token_id says which positions of input_ids hold the image")
        eng = ReasonerEngine(self.model, self.visual)
        ve, grids, deep = self._encode_images(pixel_values, image_grid_thw)
        vmask = input_ids == image_token_id
        h, _ = self.model.ar_forward(eng.embed(ids, ve, vmask), eng.positions(ids, vmask, grids), deepstack=deep,
                                     vision_mask=vmask)
        return self.model.lm_logits(h).float()

    @torch.no_grad()
    def generate(self, input_ids, pixel_values: Optional[torch.Tensor] = None, image_token_id: Optional[int] = None,
                 image_grid_thw: Optional[torch.Tensor] = None,
                 max_new_tokens: int = 64, do_sample: bool = False, temperature: float = 0.7, top_p: float = 0.8,
                 top_k: int = 20, repetition_penalty: float = 1.0, presence_penalty: float = 0.0,
                 eos_token_id: Optional[Sequence[int]] = None, seed: Optional[int] = None, **_) -> torch.Tensor:
        """input_ids [1, S] (or a list); `pixel_values` [T, 3, H, W] in [-1, 1] (one image / clip) or the patch rows
        of a `transformers` Qwen3-VL processor together with `image_grid_thw` fill the positions that hold
        `image_token_id`. Returns prompt + completion ids [1, S + n]."""
        ids = input_ids[0].tolist() if torch.is_tensor(input_ids) else list(input_ids)
        eng = ReasonerEngine(self.model, self.visual)
        ve = grids = deep = None
        if pixel_values is not None:
            ve, grids, deep = self._encode_images(pixel_values, image_grid_thw)
        dc = DecodingConfig(max_new_tokens=max_new_tokens, do_sample=do_sample, temperature=temperature, top_p=top_p,
                            top_k=top_k, repetition_penalty=repetition_penalty, presence_penalty=presence_penalty,
                            seed=seed)
        eos = () if eos_token_id is None else ([eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id))
        out, _ = eng.generate(ids, dc, eos, ve, image_token_id if ve is not None else None, grids or (), deepstack=deep)
        return torch.tensor([ids + out], dtype=torch.long)


def register() -> bool:
    """Registers the config / model with the transformers auto classes (idempotent). False without transformers."""
    if not _HAVE_HF:
        return False
    try:
        AutoConfig.register(Cosmos3ReasonerConfig.model_type, Cosmos3ReasonerConfig)
        AutoModelForCausalLM.register(Cosmos3ReasonerConfig, Cosmos3ReasonerForConditionalGeneration)
    except ValueError:
        pass  # already registered
    return True

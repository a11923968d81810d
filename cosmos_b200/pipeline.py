"""`Cosmos3OmniPipeline`: the Python API of the Generator, with the call signature of the
reference's Diffusers pipeline (reference README.md:236-275 and
cookbooks/cosmos3/generator/audiovisual/run_with_diffusers.ipynb:535-610):

    pipe = Cosmos3OmniPipeline.from_pretrained("nvidia/Cosmos3-Nano", torch_dtype=torch.bfloat16)
    pipe.scheduler = UniPCMultistepScheduler.from_config(pipe.scheduler.config, flow_shift=10.0)
    out = pipe(prompt=..., negative_prompt=..., image=None, num_frames=189, height=720, width=1280,
               fps=24, num_inference_steps=35, guidance_scale=6.0, enable_sound=False, generator=g)
    out.video, out.sound

Offline there are no published weights: `from_pretrained` loads a safetensors directory when one
is given and otherwise builds the named architecture with seeded random weights.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.nn as nn

from . import ops
from .config import (MoTConfig, SamplingConfig, get_model_config, latent_shape, resolve_size)
from .models import rope, sampler as samplers
from .models.generator import GeneratorEngine, GenState
from .models.mot import MoTModel, patchify, unpatchify
from .models.sound import SoundTokenizer
from .models.vae import CausalVideoVAE
from .utils.guardrails import Guardrails
from .utils.tokenizer import load_tokenizer


@dataclass
class SchedulerConfig:
    flow_shift: float = 10.0
    solver: str = "unipc"
    num_train_timesteps: int = 1000
    sigma_max: Optional[float] = None


class _Scheduler:
    solver = "euler"

    def __init__(self, config: Optional[SchedulerConfig] = None, **kw):
        self.config = config or SchedulerConfig()
        for k, v in kw.items():
            setattr(self.config, k, v)
        self.config.solver = self.solver

    @classmethod
    def from_config(cls, config: SchedulerConfig, **overrides):
        cfg = SchedulerConfig(**{**config.__dict__, **overrides})
        return cls(cfg)


class UniPCMultistepScheduler(_Scheduler):
    """Flow-matching UniPC multistep scheduler (`flow_shift` = sigma warp)."""
    solver = "unipc"


class FlowMatchEulerScheduler(_Scheduler):
    solver = "euler"


@dataclass
class Cosmos3Output:
    video: Any = None          # list of PIL images when num_frames == 1, else uint8 array [T, H, W, 3]
    sound: Optional[np.ndarray] = None  # [N, 2] float32 in [-1, 1] at pipe.sound_tokenizer.config.sampling_rate
    action: Optional[np.ndarray] = None
    latents: Optional[torch.Tensor] = None
    timings: Dict[str, float] = field(default_factory=dict)


RESOLUTION_TEMPLATE = " The video has a resolution of {w}x{h}."
DURATION_TEMPLATE = " The video is {sec:.1f} seconds long at {fps} frames per second."


class Cosmos3OmniPipeline:
    def __init__(self, model: MoTModel, vae: CausalVideoVAE, sound_tokenizer: SoundTokenizer, tokenizer,
                 scheduler: Optional[_Scheduler] = None, safety_checker: Optional[Guardrails] = None,
                 enable_safety_checker: bool = True, engine: Optional[GeneratorEngine] = None):
        self.transformer = model
        self.vae = vae
        self.sound_tokenizer = sound_tokenizer
        self.tokenizer = tokenizer
        self.scheduler = scheduler or UniPCMultistepScheduler()
        self.safety_checker = safety_checker if enable_safety_checker else None
        self.engine = engine or GeneratorEngine(model)
        self.action_normalizer = None   # data/vfm/action/normalization.py::ActionNormalizer, from the checkpoint's action_stats.json
        self.cfg: MoTConfig = model.cfg
        self._step_state: Optional[Tuple[GenState, SamplingConfig, torch.Tensor]] = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, name_or_path: str, torch_dtype=torch.bfloat16, device_map: Optional[str] = None,
                        safety_checker=None, enable_safety_checker: bool = True, seed: int = 0,
                        config_overrides: Optional[dict] = None, towers: Sequence[str] = ("ar", "dm"),
                        vae_widths: Sequence[int] = (64, 128, 256, 256), engine_kwargs: Optional[dict] = None,
                        layer_seed: Optional[int] = None):
        device = "cpu"
        if device_map in ("cuda", "auto") and torch.cuda.is_available():
            device = f"cuda:{torch.cuda.current_device()}"
        elif isinstance(device_map, str) and device_map.startswith("cuda"):
            device = device_map
        from .ckpt.resolve import resolve_checkpoint_dir
        ckpt_dir = resolve_checkpoint_dir(name_or_path)   # a directory, or a name with a snapshot in the local hub cache
        qwen_dir = None
        if ckpt_dir is None and Path(name_or_path).is_dir() and (Path(name_or_path) / "config.json").exists():
            doc = json.loads((Path(name_or_path) / "config.json").read_text())
            if "text_config" in doc:
                # a Hugging Face Qwen3-VL checkpoint: the Reasoner side (AR tower + vision encoder) alone
                from types import SimpleNamespace

                from .ckpt import hf_qwen3vl as hq
                qwen_dir = Path(name_or_path)
                text = SimpleNamespace(**doc["text_config"])
                text.rms_norm_eps = getattr(text, "rms_norm_eps", 1e-6)
                vis = doc.get("vision_config")
                config_overrides = {**hq.config_kwargs_from_hf(text, SimpleNamespace(**vis) if vis else None),
                                    **(config_overrides or {})}
                name_or_path, towers = "tiny", ("ar",)
        if ckpt_dir is not None and (ckpt_dir / "transformer" / "config.json").exists():
            cfg = MoTConfig(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in
                               json.loads((ckpt_dir / "transformer" / "config.json").read_text()).items()})
        else:
            cfg = get_model_config(name_or_path, **(config_overrides or {}))
        model = MoTModel(cfg, dtype=torch_dtype, device=device, towers=towers)
        model.init_weights(seed, layer_seed)
        vae = CausalVideoVAE(cfg.latent_channels, vae_widths).to(device=device, dtype=torch_dtype)
        snd = SoundTokenizer(cfg.sound_latent_dim).to(device=device, dtype=torch_dtype)
        if ckpt_dir is not None:
            from .ckpt import safetensors_io as sio
            sio.load_model(model, ckpt_dir / "transformer")
            if (ckpt_dir / "vae").is_dir():
                sio.load_into(ckpt_dir / "vae", dict(vae.state_dict()))
            if (ckpt_dir / "sound_tokenizer").is_dir():
                sio.load_into(ckpt_dir / "sound_tokenizer", dict(snd.state_dict()))
        if qwen_dir is not None:
            hq.load_checkpoint_dir(model, None, qwen_dir)
        model.eval(), vae.eval(), snd.eval()
        tok = load_tokenizer(str(ckpt_dir or qwen_dir) if (ckpt_dir or qwen_dir) else None, cfg.vocab_size)
        guard = safety_checker if safety_checker is not None else Guardrails()
        eng = GeneratorEngine(model, **(engine_kwargs or {}))
        pipe = cls(model, vae, snd, tok, None, guard, enable_safety_checker, eng)
        pipe._vision_source = ckpt_dir or qwen_dir
        if ckpt_dir is not None:
            from .data.vfm.action.normalization import STATS_FILE, ActionNormalizer
            if (ckpt_dir / STATS_FILE).exists():
                pipe.action_normalizer = ActionNormalizer.load(ckpt_dir)
        return pipe

    def vision_encoder(self):
        """The Reasoner's vision encoder for this checkpoint (built on first use, on the transformer's device and
        dtype): weights from `vision_encoder/` of a checkpoint in this package's layout or from the vision tower of a
        Qwen3-VL checkpoint directory; seeded random weights when the checkpoint has none."""
        if getattr(self, "_vit", None) is None:
            from .models.vit import VisionEncoder
            p = next(self.transformer.parameters())
            torch.manual_seed(0)
            vit = VisionEncoder(self.cfg)
            src = getattr(self, "_vision_source", None)
            if src is not None and (Path(src) / "vision_encoder").is_dir():
                from .ckpt import safetensors_io as sio
                sio.load_into(Path(src) / "vision_encoder", dict(vit.state_dict()))
            elif src is not None and (Path(src) / "config.json").exists() and not (Path(src) / "transformer").is_dir():
                from .ckpt import hf_qwen3vl as hq
                from .ckpt import safetensors_io as sio
                files = sio.tensor_files(src)
                state = {k: sio.open_reader(f).get(k) for k, f in files.items() if "visual." in k}
                if state:
                    hq.load_vision_weights(vit, state)
            self._vit = vit.to(device=p.device, dtype=p.dtype).eval()
        return self._vit

    def save_pretrained(self, out_dir) -> None:
        from .ckpt import safetensors_io as sio
        out = Path(out_dir)
        sio.save_model(self.transformer, out / "transformer")
        sio.save_sharded(dict(self.vae.state_dict()), out / "vae")
        sio.save_sharded(dict(self.sound_tokenizer.state_dict()), out / "sound_tokenizer")
        if getattr(self, "_vit", None) is not None or getattr(self, "_vision_source", None) is not None:
            sio.save_sharded(dict(self.vision_encoder().state_dict()), out / "vision_encoder")
        if self.action_normalizer is not None:
            self.action_normalizer.save(out)
        if hasattr(self.tokenizer, "hf"):  # a checkpoint's own tokenizer travels with it
            self.tokenizer.hf.save_pretrained(str(out / "tokenizer"))
        (out / "scheduler").mkdir(parents=True, exist_ok=True)
        (out / "scheduler" / "scheduler_config.json").write_text(json.dumps(self.scheduler.config.__dict__))
        (out / "model_index.json").write_text(json.dumps({
            "_class_name": "Cosmos3OmniPipeline", "transformer": "MoTModel", "vae": "CausalVideoVAE",
            "sound_tokenizer": "SoundTokenizer", "scheduler": type(self.scheduler).__name__}, indent=1))

    def to(self, device):
        self.transformer.to(device), self.vae.to(device), self.sound_tokenizer.to(device)
        self.engine = GeneratorEngine(self.transformer, cfg_group=self.engine.cfg_group)
        return self

    @property
    def device(self):
        return next(self.transformer.parameters()).device

    # ------------------------------------------------------------------ text
    def encode_text(self, text: str, max_sequence_length: Optional[int] = None) -> torch.Tensor:
        """Token ids padded / truncated to `max_sequence_length` (at most the configured 512; longer prompts
        are cut with a warning, reference README.md:389)."""
        n = self.cfg.max_text_len if not max_sequence_length else max(1, min(int(max_sequence_length), self.cfg.max_text_len))
        ids = self.tokenizer.encode(text)
        if len(ids) > n:
            import warnings
            warnings.warn(f"prompt has {len(ids)} tokens; truncated to max_sequence_length={n}", stacklevel=2)
        if hasattr(self.tokenizer, "pad_or_truncate"):
            ids = self.tokenizer.pad_or_truncate(ids, n)
        else:
            pad = self.tokenizer.pad_token_id or 0
            ids = (list(ids) + [pad] * n)[:n]
        ids = [min(int(i), self.cfg.vocab_size - 1) for i in ids]
        return torch.tensor([ids], dtype=torch.long, device=self.device)

    # ------------------------------------------------------------------ preparation
    def prepare(self, prompt: str, negative_prompt: Optional[str] = None, image=None, video=None,
                num_frames: int = 189, height: int = 720, width: int = 1280, fps: int = 24,
                num_inference_steps: int = 35, guidance_scale: float = 6.0, enable_sound: bool = False,
                add_resolution_template: bool = True, add_duration_template: bool = True,
                condition_frame_indexes: Optional[Sequence[int]] = None, action=None, domain: int = 0,
                action_dim: Optional[int] = None, denoise_action: bool = False, n_action: int = 0,
                seed: int = 0, sampling: Optional[SamplingConfig] = None,
                max_sequence_length: Optional[int] = None, sound_duration: Optional[float] = None,
                condition_video_keep: Optional[str] = None,
                negative_metadata_same: bool = False, control_video=None, control_weight: float = 1.0
                ) -> Tuple[GenState, SamplingConfig]:
        """`control_video` (a path, frames [T, H, W, 3] or a list of images: an edge / blur / depth / segmentation /
        world-scenario map of the clip to generate) makes this a video-transfer generation: the control clip is
        encoded by the tokenizer into clean latent tokens that run as a second vision stream at the target's own
        3-D rotary positions, in a third guidance branch weighted by `sampling.control_guidance * control_weight`
        (reference cookbooks/cosmos3/generator/transfer/README.md:35,98, specs/edge.json:11-22).
        `sound_duration` (seconds) overrides the sound track length, which otherwise equals the clip's
        `num_frames / fps` (reference cookbooks/cosmos3/generator/audiovisual/run_with_vllm_omni.ipynb:429).
        `condition_video_keep` says which end of an input video supplies the conditioning frames:
        "first" (default) or "last" (continue a clip from its final frames).
        `negative_metadata_same` appends the resolution / duration sentences to a plain-text negative prompt as
        well (the input spec's `negative_metadata_mode: "same"`; structured prompts carry their metadata as
        JSON keys, see io/prompt_schema.py)."""
        cfg = self.cfg
        if self.safety_checker is not None:
            self.safety_checker.check_prompt(prompt)
        suffix = ""
        if add_resolution_template:
            suffix += RESOLUTION_TEMPLATE.format(w=width, h=height)
        if add_duration_template and num_frames > 1:
            suffix += DURATION_TEMPLATE.format(sec=num_frames / float(fps), fps=fps)
        text = prompt + suffix
        if negative_metadata_same and negative_prompt and not negative_prompt.lstrip().startswith("{"):
            negative_prompt = negative_prompt + suffix
        sc = sampling or SamplingConfig(num_steps=num_inference_steps, guidance=guidance_scale,
                                        shift=self.scheduler.config.flow_shift,
                                        sigma_max=self.scheduler.config.sigma_max,
                                        scheduler=self.scheduler.config.solver, seed=seed)
        ids_c = self.encode_text(text, max_sequence_length)
        ids_u = self.encode_text(negative_prompt or "", max_sequence_length) if sc.guidance != 1.0 else None
        grid = latent_shape(cfg, num_frames, width, height)
        n_sound = 0
        if enable_sound:
            n_sound = self.sound_tokenizer.latent_frames(float(sound_duration) if sound_duration else num_frames / float(fps))
        n_act = n_action or (0 if action is None else len(action))
        st = self.engine.make_state(ids_c, ids_u, grid, n_sound, n_act, domain=domain, action_dim=action_dim, fps=fps)
        s_dm = st.pos.shape[1]
        feat = max(cfg.patch_dim, cfg.sound_latent_dim if n_sound else 0, action_dim or 0 if n_act else 0)
        cond = torch.zeros(s_dm, dtype=torch.bool, device=self.device)
        clean = torch.zeros(1, s_dm, feat, dtype=torch.float32, device=self.device)
        tokens_per_frame = (grid[1] // cfg.patch_hw) * (grid[2] // cfg.patch_hw)
        vdt = next(self.vae.parameters()).dtype
        frames = None
        if image is not None:
            frames = _to_frames(image, width, height)[:1]
            condition_frame_indexes = [0] if condition_frame_indexes is None else condition_frame_indexes
        elif video is not None:
            frames = _to_frames(video, width, height)
            condition_frame_indexes = list(condition_frame_indexes or [0])
        if frames is not None:
            n_lat = max(condition_frame_indexes) + 1
            n_pix = 1 + (n_lat - 1) * cfg.vae_t_compress
            if condition_video_keep not in (None, "first", "last"):
                raise ValueError(f"condition_video_keep must be 'first' or 'last', got {condition_video_keep!r}")
            fr = frames[-n_pix:] if condition_video_keep == "last" else frames[:n_pix]
            if fr.shape[0] < n_pix:
                fr = np.concatenate([fr, np.repeat(fr[-1:], n_pix - fr.shape[0], 0)])
            x = CausalVideoVAE.from_uint8(torch.from_numpy(np.array(fr))[None].to(self.device)).to(vdt)
            z = self._encode_video(x)
            ztok = patchify(z, cfg)[0]
            for li in condition_frame_indexes:
                a, b = li * tokens_per_frame, (li + 1) * tokens_per_frame
                cond[a:b] = True
                clean[0, a:b, :cfg.patch_dim] = ztok[a:b]
        if action is not None and not denoise_action:
            if self.action_normalizer is not None:      # per-embodiment standardisation (data/vfm/action/normalization.py)
                action = self.action_normalizer.normalize(action, cfg.action_domains[domain])
            a = torch.as_tensor(np.asarray(action), dtype=torch.float32, device=self.device)
            off = st.n_video + st.n_sound
            cond[off:off + a.shape[0]] = True
            clean[0, off:off + a.shape[0], :a.shape[1]] = a
        if control_video is not None:
            if n_sound or n_act:
                raise ValueError("video transfer (a control clip) generates vision only")
            n_pix = 1 + (grid[0] - 1) * cfg.vae_t_compress
            cf = _to_frames(control_video, width, height)[:n_pix]
            if cf.shape[0] < n_pix:
                cf = np.concatenate([cf, np.repeat(cf[-1:], n_pix - cf.shape[0], 0)])
            cx = CausalVideoVAE.from_uint8(torch.from_numpy(np.array(cf))[None].to(self.device)).to(vdt)
            cz = self._encode_video(cx)
            ctok = patchify(cz, cfg)                       # [1, all video tokens, patch_dim]
            a = st.shard_start
            st.control_tokens = ctok[:, a:a + st.n_video].contiguous()   # this rank's context-parallel shard
            st.control_weight = float(control_weight)
        if cond.any():
            st.cond_mask, st.clean_tokens = cond, clean
        return st, sc

    # ------------------------------------------------------------------ step-wise public API
    @torch.no_grad()
    def begin(self, st: GenState, sc: SamplingConfig, noise: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Starts a step-wise generation; returns the initial fp32 latent tokens [1, S, F]."""
        s_dm = st.pos.shape[1]
        total = st.total_tokens or s_dm
        f = st.clean_tokens.shape[-1] if st.clean_tokens is not None else self.cfg.patch_dim
        if noise is None:
            g = torch.Generator(device=self.device)
            g.manual_seed(sc.seed)
            noise = torch.randn(1, total, f, generator=g, device=self.device, dtype=torch.float32)
        if noise.shape[1] != s_dm:  # context-parallel shard of the full-sequence noise
            noise = noise[:, st.shard_start:st.shard_start + s_dm].contiguous()
        sig = samplers.shifted_sigmas(sc.num_steps, sc.shift, sc.sigma_max, device="cpu")
        self._step_state = (st, sc, sig)
        self._sampler = samplers.make_sampler(sc.scheduler, sig)
        return noise * float(sig[0]) if sc.sigma_max is not None else noise

    @torch.no_grad()
    def step(self, latents: torch.Tensor, i: int) -> torch.Tensor:
        """Advances device-resident latents by denoise step i."""
        st, sc, sig = self._step_state
        smp = self._sampler
        smp.i = i
        return self.engine.denoise_step(latents, float(sig[i]), float(sig[i + 1]), st, sc, smp)

    @torch.no_grad()
    def step_from_host(self, latents_host: torch.Tensor, i: int, out_host: Optional[torch.Tensor] = None
                       ) -> torch.Tensor:
        """One denoise step on host-resident latents: pinned host -> device copy, the guided step
        on the GPU(s), and the updated latents copied back to (pinned) host memory."""
        dev_lat = latents_host.to(self.device, non_blocking=True)
        new = self.step(dev_lat, i)
        if out_host is None:
            out_host = torch.empty_like(latents_host)
        out_host.copy_(new, non_blocking=True)
        torch.cuda.current_stream().synchronize() if self.device.type == "cuda" else None
        return out_host

    def _cl_decoder(self):
        """The sm_100a tokenizer decoder when the VAE is on CUDA in bf16 with 64-multiple widths."""
        if getattr(self, "_cl", None) is not None:
            return self._cl
        p0 = next(self.vae.parameters())
        widths_ok = all(m.weight.shape[0] % 64 == 0 for m in [self.vae.dec_in] + [u.conv for u in self.vae.dec_up])
        if p0.is_cuda and p0.dtype == torch.bfloat16 and widths_ok and ops.load_extension() and \
                self.vae.dec_out.weight.shape[1] == 64:
            from .models.vae_cuda import CLDecoder
            self._cl = CLDecoder(self.vae)
            return self._cl
        return None

    def _encode_video(self, x: torch.Tensor) -> torch.Tensor:
        """[1, 3, T, H, W] in [-1, 1] -> latent mean [1, C, 1 + (T - 1) / 4, H / 8, W / 8] (fp32). On CUDA in bf16 with
        64-multiple widths the implicit-GEMM encoder (`models/vae_cuda.py::CLEncoder`), else the PyTorch modules."""
        n_pix = x.shape[2]
        enc = getattr(self, "_cl_enc", None)
        if enc is None:
            p0 = next(self.vae.parameters())
            convs = [self.vae.enc_in] + [d.conv for d in self.vae.enc_down]
            ok = (p0.is_cuda and p0.dtype == torch.bfloat16 and ops.get_backend() != "library" and
                  all(m.weight.shape[0] % 64 == 0 for m in convs) and ops.load_extension())
            if ok:
                from .models.vae_cuda import CLEncoder
                enc = self._cl_enc = CLEncoder(self.vae)
            else:
                self._cl_enc = enc = False
        if enc and x.shape[3] % 8 == 0 and x.shape[4] % 8 == 0:
            return enc.encode(x, chunk_frames=8)
        with torch.no_grad():
            return self.vae.encode(x, chunk_frames=4 if n_pix > 1 else None).float()

    def gather_tokens(self, tokens: torch.Tensor, st: GenState) -> torch.Tensor:
        """All-gathers context-parallel token shards into the full sequence (no-op without cp)."""
        ctx = self.engine.ctx
        if getattr(ctx, "cp", 1) == 1 or not st.total_tokens or st.total_tokens == tokens.shape[1]:
            return tokens
        import torch.distributed as dist
        parts = [torch.empty_like(tokens) for _ in range(ctx.cp)]
        dist.all_gather(parts, tokens.contiguous(), group=ctx.group)
        return torch.cat(parts, dim=1)

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def decode(self, tokens: torch.Tensor, st: GenState, chunk_latents: Optional[int] = 4):
        cfg = self.cfg
        vdt = next(self.vae.parameters()).dtype
        tokens = self.gather_tokens(tokens, st)
        n_video = st.n_video if not st.total_tokens or st.total_tokens == st.pos.shape[1] else st.total_tokens
        z = unpatchify(tokens[:, :n_video, :cfg.patch_dim], cfg, st.grid).to(vdt)
        cl = self._cl_decoder()
        if cl is not None:
            # tensor-core implicit-GEMM decoder on padded channels-last volumes (2 latent frames per chunk)
            frames = cl.decode(z, chunk_latents=2)[0].cpu().numpy()
        else:
            video = self.vae.decode(z, chunk_latents=chunk_latents if st.grid[0] > (chunk_latents or 0) else None)
            frames = CausalVideoVAE.to_uint8(video)[0].cpu().numpy()
        sound = None
        if st.n_sound:
            lat = tokens[:, st.n_video:st.n_video + st.n_sound, :cfg.sound_latent_dim]
            sound = self.sound_tokenizer.decode(lat.to(vdt))[0].float().cpu().numpy()
        action = None
        if st.n_action:
            off = st.n_video + st.n_sound
            action = tokens[0, off:off + st.n_action, :st.action_dim].float().cpu().numpy()
            if self.action_normalizer is not None and getattr(st, "domain", None) is not None:
                action = self.action_normalizer.denormalize(action, self.cfg.action_domains[int(st.domain)])
        return frames, sound, action

    # ------------------------------------------------------------------ long videos
    @torch.no_grad()
    def forward_dynamics_rollout(self, image, actions, action_chunk_size: int = 16, domain: int = 0, prompt: str = "",
                                 height: int = 480, width: int = 832, fps: int = 15, seed: int = 0, callback=None,
                                 **call_kw) -> Cosmos3Output:
        """Autoregressive forward dynamics over a long action sequence, in one process: the actions [N, D] are cut
        into chunks of `action_chunk_size` (N must be a multiple of it), chunk k starts from the last frame that chunk
        k - 1 produced and uses seed + k, and the clips are joined without repeating the shared frame: 1 + N frames in
        all. This is the loop the reference's DROID / UMI notebooks run on the client side (reference
        cookbooks/cosmos3/generator/action/run_fd_with_cosmos_framework.ipynb, the "autoregressive chunks" cells)."""
        acts = np.asarray(actions, dtype=np.float32)
        if acts.ndim != 2 or acts.shape[0] == 0 or acts.shape[0] % action_chunk_size:
            raise ValueError(f"actions must be [N, D] with N a positive multiple of action_chunk_size={action_chunk_size}, "
                             f"got {acts.shape}")
        frames, timings, cur = [], {}, image
        n_chunks = acts.shape[0] // action_chunk_size
        for k in range(n_chunks):
            chunk = acts[k * action_chunk_size:(k + 1) * action_chunk_size]
            out = self(prompt=prompt, image=cur, num_frames=action_chunk_size + 1, height=height, width=width, fps=fps,
                       action=chunk, domain=domain, action_dim=acts.shape[1], output_type="np",
                       generator=torch.Generator().manual_seed(seed + k), **call_kw)
            frames.append(out.video if k == 0 else out.video[1:])
            cur = out.video[-1]
            for name, v in out.timings.items():
                timings[name] = timings.get(name, 0.0) + v
            if callback is not None:
                callback(k, n_chunks)
        return Cosmos3Output(video=np.concatenate(frames), timings=timings)

    def generate_chunked(self, prompt: str, negative_prompt: Optional[str] = None, video=None,
                         num_frames: int = 121, height: int = 720, width: int = 1280, fps: int = 24,
                         frames_per_chunk: int = 121, num_conditional_frames: int = 1,
                         num_first_chunk_conditional_frames: int = 0, sampling: Optional[SamplingConfig] = None,
                         callback=None, **call_kw) -> Cosmos3Output:
        """Generates `num_frames` frames chunk by chunk (`num_video_frames_per_chunk`,
        `num_conditional_frames`, `num_first_chunk_conditional_frames` of the reference's transfer
        specs, cookbooks/cosmos3/generator/transfer/specs/edge.json:11-13). The first chunk is
        conditioned on the leading frames of `video` (if any), every later chunk on the last
        `num_conditional_frames` frames generated so far, which enter as clean latent frames; the
        overlap is dropped from the output. Each chunk uses seed + chunk index."""
        import dataclasses

        tc = self.cfg.vae_t_compress
        n_first = num_first_chunk_conditional_frames if video is not None else 0
        plan = _chunk_plan(num_frames, frames_per_chunk, n_first, num_conditional_frames, tc)
        src = _to_frames(video, width, height) if video is not None else None
        ctrl_src = call_kw.pop("control_video", None)
        ctrl_all = _to_frames(ctrl_src, width, height) if ctrl_src is not None else None
        done = 0   # output frames produced so far = position of the next chunk's first new frame in the clip
        frames_out: List[np.ndarray] = []
        sounds, timings = [], {}
        tail = None
        last = None
        for k, (c, new, total) in enumerate(plan):
            cond = None
            if k == 0 and c:
                cond = src[:c]
            elif k > 0 and c:
                cond = tail[-c:]
            kw = dict(call_kw)
            if cond is not None:
                kw["condition_frame_indexes"] = list(range(1 + (c - 1) // tc))
            if ctrl_all is not None:
                # the chunk covers clip frames [done - c, done - c + total): its control frames are the same range
                lo = max(0, done - c)
                seg = ctrl_all[lo:lo + total]
                if seg.shape[0] == 0:
                    seg = ctrl_all[-1:]
                kw["control_video"] = seg
            sc = dataclasses.replace(sampling, seed=sampling.seed + k) if sampling is not None else None
            if sc is None and "generator" not in kw:
                kw["generator"] = torch.Generator().manual_seed(k)
            last = self(prompt, negative_prompt, video=cond, num_frames=total, height=height, width=width, fps=fps,
                        sampling=sc, callback=callback, **kw)
            fr = np.asarray(last.video)
            frames_out.append(fr[c:c + new])
            done += new
            tail = fr[:c + new]
            if last.sound is not None:
                sounds.append(np.asarray(last.sound))
            for name, v in last.timings.items():
                timings[name] = timings.get(name, 0.0) + v
        timings["chunks"] = len(plan)
        sound = np.concatenate(sounds, axis=0) if sounds else None
        return Cosmos3Output(video=np.concatenate(frames_out, axis=0), sound=sound, action=last.action,
                             latents=last.latents, timings=timings)

    # ------------------------------------------------------------------ __call__
    @torch.no_grad()
    def __call__(self, prompt: str, negative_prompt: Optional[str] = None, image=None, video=None,
                 num_frames: int = 189, height: int = 720, width: int = 1280, fps: int = 24,
                 num_inference_steps: int = 35, guidance_scale: float = 6.0, enable_sound: bool = False,
                 add_resolution_template: bool = True, add_duration_template: bool = True,
                 generator: Optional[torch.Generator] = None, output_type: str = "pil",
                 sampling: Optional[SamplingConfig] = None, callback=None, **prep_kw) -> Cosmos3Output:
        from .utils.obs import nvtx_range
        t0 = time.perf_counter()
        seed = int(generator.initial_seed()) if generator is not None else (sampling.seed if sampling else 0)
        with nvtx_range("generate/prepare"):
            st, sc = self.prepare(prompt, negative_prompt, image, video, num_frames, height, width, fps,
                                  num_inference_steps, guidance_scale, enable_sound, add_resolution_template,
                                  add_duration_template, seed=seed, sampling=sampling, **prep_kw)
        t1 = time.perf_counter()
        x = self.begin(st, sc)
        for i in range(sc.num_steps):
            with nvtx_range(f"generate/step{i}"):
                x = self.step(x, i)
            if callback is not None:
                callback(i, sc.num_steps)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
            ops.check_status()
        t2 = time.perf_counter()
        if output_type == "latent":
            return Cosmos3Output(latents=x, timings={"prepare_s": t1 - t0, "sample_s": t2 - t1})
        with nvtx_range("generate/decode"):
            frames, sound, action = self.decode(x, st)
        if self.safety_checker is not None:
            frames = self.safety_checker.blur_faces(frames)
        t3 = time.perf_counter()
        video_out: Any = frames
        if output_type not in ("pil", "np", "latent"):
            raise ValueError("output_type must be 'pil', 'np' or 'latent'")
        # "pil" (the default, as in the reference's Diffusers surface): a single image comes back as [PIL.Image],
        # so `out.video[0].save(path)` works; a clip is a uint8 array [T, H, W, 3] either way
        if num_frames == 1 and output_type == "pil":
            from PIL import Image
            video_out = [Image.fromarray(frames[0])]
        return Cosmos3Output(video=video_out, sound=sound, action=action, latents=x,
                             timings={"prepare_s": t1 - t0, "sample_s": t2 - t1, "decode_s": t3 - t2})


def _chunk_plan(num_frames: int, frames_per_chunk: int, n_cond_first: int, n_cond: int, t_compress: int
                ) -> List[Tuple[int, int, int]]:
    """(conditioning frames, new frames, pixel frames generated) per chunk for a long video: every
    chunk holds at most `frames_per_chunk` pixel frames, the first `n_cond` (first chunk:
    `n_cond_first`) of them repeat the tail of what exists already, and the generated length is
    rounded up to the tokenizer's 1 + k * t_compress frame grid."""
    if frames_per_chunk <= max(n_cond, n_cond_first):
        raise ValueError("num_video_frames_per_chunk must exceed the number of conditional frames")
    plan, done, k = [], 0, 0
    while done < num_frames:
        c = n_cond_first if k == 0 else n_cond
        new = min(frames_per_chunk - c, num_frames - done)
        total = c + new
        total = 1 + -(-(total - 1) // t_compress) * t_compress
        plan.append((c, new, total))
        done += new
        k += 1
    return plan


def _to_frames(media, width: int, height: int) -> np.ndarray:
    """PIL image / uint8 array [H, W, 3] or [T, H, W, 3] / path -> uint8 [T, height, width, 3]."""
    from PIL import Image
    from .io import media as mio

    if isinstance(media, (str, Path)):
        return mio.read_video(media, size=(width, height))[0]
    if isinstance(media, Image.Image):
        return np.asarray(mio._resize_center_crop(media.convert("RGB"), (width, height)))[None]
    arr = np.asarray(media)
    if arr.ndim == 3:
        arr = arr[None]
    if (arr.shape[2], arr.shape[1]) != (width, height):
        arr = np.stack([np.asarray(mio._resize_center_crop(Image.fromarray(f), (width, height))) for f in arr])
    return arr.astype(np.uint8)

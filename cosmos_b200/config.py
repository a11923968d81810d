"""Configuration dataclasses: model shapes, parallel layout, sampling recipe.

The reference publishes no model config file; tower shapes follow the public Qwen3-VL text
configs that the reference says its Reasoner is based on (reference README.md:286; model
sizes README.md:79-85: Nano 16B = 2 x 8B towers, Super 64B = 2 x 32B towers).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Dict, List, Optional, Tuple


@dataclass
class MoTConfig:
    name: str = "tiny"
    d_model: int = 512
    n_layers: int = 4
    n_heads: int = 8
    n_kv_heads: int = 8
    head_dim: int = 64
    ffn_dim: int = 2048
    vocab_size: int = 32000
    rope_theta: float = 5.0e5
    mrope_section: Tuple[int, int, int] = (12, 10, 10)  # (t, h, w) frequency counts, sum = head_dim / 2
    rms_eps: float = 1e-6
    qk_norm: bool = True
    share_attn_proj: bool = False  # True: AR and DM towers use the same QKV/O projection weights
    # DM side
    latent_channels: int = 16
    patch_t: int = 1
    patch_hw: int = 2
    vae_t_compress: int = 4
    vae_s_compress: int = 8
    t_embed_dim: int = 256
    sound_latent_dim: int = 64      # channels of one audio latent frame
    action_dim_max: int = 64        # padded per-domain raw action dim
    action_domains: Tuple[str, ...] = ("av", "droid_lerobot", "umi", "bridge_orig_lerobot", "camera_pose")
    # AR side vision encoder (ViT) — Qwen3-VL conventions
    vit_depth: int = 2
    vit_hidden: int = 128
    vit_heads: int = 4
    vit_patch: int = 16
    vit_temporal_patch: int = 2
    vit_spatial_merge: int = 2
    # ViT block indexes whose features are merged and added to the hidden states of the first AR layers
    # (DeepStack of the Qwen3-VL family the Reasoner follows; () = off)
    vit_deepstack: Tuple[int, ...] = ()
    vit_ffn: int = 0          # MLP width of a ViT block; 0 = 4 x vit_hidden
    vit_pos_side: int = 48    # the learned position table covers vit_pos_side x vit_pos_side patches
    max_text_len: int = 512
    init_std: float = 0.02

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def patch_dim(self) -> int:
        return self.latent_channels * self.patch_t * self.patch_hw * self.patch_hw

    def tower_params(self) -> int:
        """Parameter count of one tower's transformer body (no embeddings)."""
        per_layer = (self.qkv_dim * self.d_model + self.d_model * self.q_dim
                     + 3 * self.ffn_dim * self.d_model + 2 * self.d_model + 2 * self.head_dim)
        return per_layer * self.n_layers

    def to_dict(self) -> Dict:
        return asdict(self)


def tiny_config(**kw) -> MoTConfig:
    """4 layers, d=512, 8 heads of 64, MLP 4x, 32k vocab: the CPU/gloo plumbing model."""
    return replace(MoTConfig(), **kw)


def tiny128_config(**kw) -> MoTConfig:
    """Small model with head_dim 128 so that every CUDA kernel (attention included) is on its path."""
    base = MoTConfig(name="tiny128", d_model=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128,
                     ffn_dim=1024, vocab_size=4096, mrope_section=(24, 20, 20))
    return replace(base, **kw)


def nano_config(**kw) -> MoTConfig:
    """Cosmos3-Nano stand-in: two Qwen3-VL-8B-shaped towers (16.4 B parameters)."""
    base = MoTConfig(name="Cosmos3-Nano", d_model=4096, n_layers=36, n_heads=32, n_kv_heads=8, head_dim=128,
                     ffn_dim=12288, vocab_size=151936, mrope_section=(24, 20, 20),
                     vit_depth=27, vit_hidden=1152, vit_heads=16, vit_ffn=4304, vit_deepstack=(8, 16, 24))
    return replace(base, **kw)


def super_config(**kw) -> MoTConfig:
    """Cosmos3-Super stand-in: two Qwen3-VL-32B-shaped towers (65.5 B parameters)."""
    base = MoTConfig(name="Cosmos3-Super", d_model=5120, n_layers=64, n_heads=64, n_kv_heads=8, head_dim=128,
                     ffn_dim=25600, vocab_size=151936, mrope_section=(24, 20, 20),
                     vit_depth=27, vit_hidden=1152, vit_heads=16, vit_ffn=4304, vit_deepstack=(8, 16, 24))
    return replace(base, **kw)


MODEL_REGISTRY = {
    "tiny": tiny_config,
    "tiny128": tiny128_config,
    "Cosmos3-Nano": nano_config,
    "Cosmos3-Super": super_config,
    "nvidia/Cosmos3-Nano": nano_config,
    "nvidia/Cosmos3-Super": super_config,
}


def get_model_config(name: str, **kw) -> MoTConfig:
    key = name.rstrip("/").split("/")[-1] if name not in MODEL_REGISTRY else name
    if key not in MODEL_REGISTRY:
        raise KeyError(f"unknown model '{name}'; known: {sorted(MODEL_REGISTRY)}")
    return MODEL_REGISTRY[key](**kw)


# --------------------------------------------------------------------------- resolution tables
# Reference README.md:106 and inference_benchmarks.md:39: 720p = 1280x720, 480p = 832x480, 256p = 320x192.
RESOLUTIONS_16_9 = {"720": (1280, 720), "480": (832, 480), "256": (320, 192)}
ASPECT_RATIOS = ("16,9", "4,3", "1,1", "3,4", "9,16")


def resolve_size(resolution: str, aspect_ratio: str = "16,9") -> Tuple[int, int]:
    """(width, height) in pixels, multiples of 16, for a resolution tier and aspect ratio."""
    resolution = str(resolution)
    if resolution not in RESOLUTIONS_16_9:
        raise ValueError(f"resolution must be one of {sorted(RESOLUTIONS_16_9)}, got {resolution!r}")
    if aspect_ratio not in ASPECT_RATIOS:
        raise ValueError(f"aspect_ratio must be one of {ASPECT_RATIOS}, got {aspect_ratio!r}")
    w169, h169 = RESOLUTIONS_16_9[resolution]
    if aspect_ratio == "16,9":
        return w169, h169
    if aspect_ratio == "9,16":
        return h169, w169
    aw, ah = (int(v) for v in aspect_ratio.split(","))
    area = w169 * h169
    h = (area * ah / aw) ** 0.5
    w = h * aw / ah
    r16 = lambda v: max(16, int(round(v / 16)) * 16)  # noqa: E731
    return r16(w), r16(h)


def latent_shape(cfg: MoTConfig, num_frames: int, width: int, height: int) -> Tuple[int, int, int]:
    """(T, H, W) of the VAE latent for a clip (first frame alone, then groups of vae_t_compress)."""
    t = (num_frames - 1) // cfg.vae_t_compress + 1
    return t, height // cfg.vae_s_compress, width // cfg.vae_s_compress


def video_token_count(cfg: MoTConfig, num_frames: int, width: int, height: int) -> int:
    t, h, w = latent_shape(cfg, num_frames, width, height)
    return (t // cfg.patch_t) * (h // cfg.patch_hw) * (w // cfg.patch_hw)


# --------------------------------------------------------------------------- parallel layout
@dataclass
class ParallelConfig:
    """Mesh degrees; their product must equal the world size (reference README.md:321)."""
    dp_replicate: int = 1
    dp_shard: int = 1
    cp: int = 1
    cfgp: int = 1
    tp: int = 1
    cp_mode: str = "ulysses"  # or "ring"

    @property
    def world(self) -> int:
        return self.dp_replicate * self.dp_shard * self.cp * self.cfgp * self.tp

    def validate(self, world_size: int) -> None:
        for k in ("dp_replicate", "dp_shard", "cp", "cfgp", "tp"):
            if getattr(self, k) < 1:
                raise ValueError(f"{k} must be >= 1")
        if self.cfgp not in (1, 2):
            raise ValueError("cfgp must be 1 or 2 (cond / uncond branches)")
        if self.world != world_size:
            raise ValueError(f"product of parallel degrees {self.world} != world size {world_size}")
        if self.cp_mode not in ("ulysses", "ring"):
            raise ValueError("cp_mode must be 'ulysses' or 'ring'")


def preset_parallelism(preset: str, world_size: int, use_cfg: bool = True, n_kv_heads: int = 8) -> ParallelConfig:
    """`latency`: all GPUs on one sample (CFG-parallel x context-parallel).
    `throughput`: replicate the model and give each replica its own samples
    (reference: cookbooks/cosmos3/generator/transfer/README.md:51,
    audiovisual/run_with_cosmos_framework.ipynb:529-533)."""
    if preset == "throughput":
        return ParallelConfig(dp_replicate=world_size)
    if preset != "latency":
        raise ValueError("parallelism preset must be 'latency' or 'throughput'")
    cfgp = 2 if (use_cfg and world_size % 2 == 0 and world_size >= 2) else 1
    cp = world_size // cfgp
    mode = "ulysses" if cp <= n_kv_heads and n_kv_heads % cp == 0 else "ring"
    return ParallelConfig(cp=cp, cfgp=cfgp, cp_mode=mode)


# --------------------------------------------------------------------------- sampling recipe
@dataclass
class SamplingConfig:
    """Generator defaults (reference README.md:249-263; audiovisual/README.md:43-48)."""
    num_steps: int = 35
    guidance: float = 6.0
    shift: float = 10.0
    sigma_max: Optional[float] = None
    guidance_interval: Tuple[float, float] = (0.0, 1000.0)
    normalize_cfg: bool = False
    control_guidance: Optional[float] = None
    scheduler: str = "euler"  # or "unipc"
    seed: int = 0


@dataclass
class DecodingConfig:
    """Reasoner decoding defaults (reference README.md:159-167)."""
    max_new_tokens: int = 4096
    do_sample: bool = True
    temperature: float = 0.7
    top_p: float = 0.8
    top_k: int = 20
    repetition_penalty: float = 1.0
    presence_penalty: float = 1.5
    seed: Optional[int] = None

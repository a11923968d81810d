"""Weights of a Qwen3-VL model <-> the Reasoner side of this framework (AR tower, embeddings, LM head, ViT).

The reference's Reasoner is "Qwen3-VL-based" (reference README.md:286) and its AR tower has the Qwen3-VL text shapes
(Nano = Qwen3-VL-8B, Super = Qwen3-VL-32B). With the tensors mapped by this module the AR tower reproduces the hidden
states of `transformers`' `Qwen3VLTextModel` (interleaved 3-D mRoPE, q/k RMS-norm, DeepStack injection included) and the
vision encoder reproduces `Qwen3VLVisionModel` (tests/test_hf_parity_cpu.py), so a Reasoner can be initialised from
a Qwen3-VL checkpoint and exported back to that layout for other runtimes.

Name map (HF -> here). Text: `embed_tokens.weight` -> `embed`; `norm.weight` -> `ar_norm`; `lm_head.weight` -> `lm_head`
(tied to the embedding when absent); per layer `input_layernorm` -> `norm1`, `q_proj | k_proj | v_proj` stacked ->
`wqkv`, `q_norm`, `k_norm`, `o_proj` -> `wo`, `post_attention_layernorm` -> `norm2`, `gate_proj | up_proj` stacked ->
`w_gate_up`, `down_proj` -> `w_down`. Vision: `patch_embed.proj` (conv3d kernel) -> `patch` (flattened), `pos_embed` ->
`pos`, blocks `norm1/norm2/attn.qkv/attn.proj/mlp.linear_fc1/mlp.linear_fc2` -> `n1/n2/qkv/proj/fc1/fc2`, `merger.{norm,
linear_fc1,linear_fc2}` -> `norm`, `merge.0`, `merge.2`, `deepstack_merger_list.k.*` -> `deepstack_norm.k`,
`deepstack_merge.k.{0,2}`. Key prefixes `model.`, `language_model.`, `model.language_model.`, `visual.`,
`model.visual.` are accepted.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..config import MoTConfig

_TEXT_PREFIXES = ("model.language_model.", "language_model.model.", "language_model.", "model.", "")
_VISION_PREFIXES = ("model.visual.", "visual.", "vision_model.", "")


def config_kwargs_from_hf(text_config, vision_config=None) -> Dict[str, object]:
    """MoTConfig fields that follow from a Qwen3-VL (text, vision) config pair."""
    rp = getattr(text_config, "rope_parameters", None) or getattr(text_config, "rope_scaling", None) or {}
    kw: Dict[str, object] = dict(
        d_model=text_config.hidden_size, n_layers=text_config.num_hidden_layers, n_heads=text_config.num_attention_heads,
        n_kv_heads=text_config.num_key_value_heads,
        head_dim=getattr(text_config, "head_dim", None) or text_config.hidden_size // text_config.num_attention_heads,
        ffn_dim=text_config.intermediate_size, vocab_size=text_config.vocab_size, rms_eps=text_config.rms_norm_eps,
        rope_theta=float(rp.get("rope_theta", getattr(text_config, "rope_theta", 5e5))),
        mrope_section=tuple(rp.get("mrope_section", (24, 20, 20))))
    if vision_config is not None:
        side = int(round(vision_config.num_position_embeddings ** 0.5))
        kw.update(vit_depth=vision_config.depth, vit_hidden=vision_config.hidden_size, vit_heads=vision_config.num_heads,
                  vit_ffn=vision_config.intermediate_size, vit_patch=vision_config.patch_size,
                  vit_temporal_patch=vision_config.temporal_patch_size, vit_spatial_merge=vision_config.spatial_merge_size,
                  vit_pos_side=side, vit_deepstack=tuple(vision_config.deepstack_visual_indexes))
    return kw


def _strip(state: Mapping[str, torch.Tensor], prefixes, probe: str) -> Dict[str, torch.Tensor]:
    for p in prefixes:
        if p + probe in state:
            return {k[len(p):]: v for k, v in state.items() if k.startswith(p)}
    raise KeyError(f"no '{probe}' under any of the prefixes {prefixes}")


@torch.no_grad()
def load_text_weights(model, state: Mapping[str, torch.Tensor], strict: bool = True) -> None:
    """Copies a Qwen3-VL text model's tensors into `model` (a MoTModel with an AR tower)."""
    cfg: MoTConfig = model.cfg
    sd = _strip(state, _TEXT_PREFIXES, "embed_tokens.weight")
    if sd["embed_tokens.weight"].shape != model.embed.shape:
        raise ValueError(f"embedding shape {tuple(sd['embed_tokens.weight'].shape)} != {tuple(model.embed.shape)}")
    model.embed.copy_(sd["embed_tokens.weight"])
    model.ar_norm.copy_(sd["norm.weight"])
    head = state.get("lm_head.weight", state.get("model.lm_head.weight"))
    model.lm_head.copy_(sd["embed_tokens.weight"] if head is None else head)
    n_hf = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
    if strict and n_hf != cfg.n_layers:
        raise ValueError(f"checkpoint has {n_hf} layers, the model {cfg.n_layers}")
    for i, layer in enumerate(model.ar.layers):
        g = lambda k: sd[f"layers.{i}.{k}.weight"]  # noqa: E731
        v = layer.views()
        v["norm1"].copy_(g("input_layernorm"))
        v["wqkv"].copy_(torch.cat([g("self_attn.q_proj"), g("self_attn.k_proj"), g("self_attn.v_proj")]))
        v["q_norm"].copy_(g("self_attn.q_norm"))
        v["k_norm"].copy_(g("self_attn.k_norm"))
        v["wo"].copy_(g("self_attn.o_proj"))
        v["norm2"].copy_(g("post_attention_layernorm"))
        v["w_gate_up"].copy_(torch.cat([g("mlp.gate_proj"), g("mlp.up_proj")]))
        v["w_down"].copy_(g("mlp.down_proj"))


def export_text_weights(model, prefix: str = "model.language_model.") -> Dict[str, torch.Tensor]:
    """The AR tower in the Qwen3-VL text layout (inverse of `load_text_weights`)."""
    cfg: MoTConfig = model.cfg
    out = {prefix + "embed_tokens.weight": model.embed.detach().clone(), prefix + "norm.weight": model.ar_norm.detach().clone(),
           "lm_head.weight": model.lm_head.detach().clone()}
    qd, kd = cfg.q_dim, cfg.n_kv_heads * cfg.head_dim
    for i, layer in enumerate(model.ar.layers):
        v = {k: t.detach().clone() for k, t in layer.views().items()}
        p = f"{prefix}layers.{i}."
        out[p + "input_layernorm.weight"] = v["norm1"]
        out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"], out[p + "self_attn.v_proj.weight"] = \
            v["wqkv"][:qd], v["wqkv"][qd:qd + kd], v["wqkv"][qd + kd:]
        out[p + "self_attn.q_norm.weight"], out[p + "self_attn.k_norm.weight"] = v["q_norm"], v["k_norm"]
        out[p + "self_attn.o_proj.weight"] = v["wo"]
        out[p + "post_attention_layernorm.weight"] = v["norm2"]
        out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = v["w_gate_up"][:cfg.ffn_dim], v["w_gate_up"][cfg.ffn_dim:]
        out[p + "mlp.down_proj.weight"] = v["w_down"]
    return out


_VISION_BLOCK = {"norm1": "n1", "norm2": "n2", "attn.qkv": "qkv", "attn.proj": "proj", "mlp.linear_fc1": "fc1",
                 "mlp.linear_fc2": "fc2"}


def vision_state_from_hf(state: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """A Qwen3-VL vision tower's tensors under this package's `VisionEncoder` names."""
    sd = _strip(state, _VISION_PREFIXES, "patch_embed.proj.weight")
    out: Dict[str, torch.Tensor] = {"patch.weight": sd["patch_embed.proj.weight"].flatten(1), "patch.bias": sd["patch_embed.proj.bias"],
                                    "pos": sd["pos_embed.weight"]}
    for k, t in sd.items():
        parts = k.split(".")
        if parts[0] == "blocks":
            mid, leaf = ".".join(parts[2:-1]), parts[-1]
            out[f"blocks.{parts[1]}.{_VISION_BLOCK[mid]}.{leaf}"] = t
        elif parts[0] == "merger":
            name = {"norm": "norm", "linear_fc1": "merge.0", "linear_fc2": "merge.2"}[parts[1]]
            out[f"{name}.{parts[2]}"] = t
        elif parts[0] == "deepstack_merger_list":
            name = {"norm": f"deepstack_norm.{parts[1]}", "linear_fc1": f"deepstack_merge.{parts[1]}.0",
                    "linear_fc2": f"deepstack_merge.{parts[1]}.2"}[parts[2]]
            out[f"{name}.{parts[3]}"] = t
    return out


def export_vision_weights(vit, prefix: str = "model.visual.") -> Dict[str, torch.Tensor]:
    """The vision encoder in the Qwen3-VL vision layout (inverse of `vision_state_from_hf`)."""
    c = vit.cfg
    inv_block = {v: k for k, v in _VISION_BLOCK.items()}
    out: Dict[str, torch.Tensor] = {}
    for k, t in vit.state_dict().items():
        t = t.detach().clone()
        parts = k.split(".")
        if k == "patch.weight":
            out[prefix + "patch_embed.proj.weight"] = t.view(t.shape[0], 3, c.vit_temporal_patch, c.vit_patch, c.vit_patch)
        elif k == "patch.bias":
            out[prefix + "patch_embed.proj.bias"] = t
        elif k == "pos":
            out[prefix + "pos_embed.weight"] = t
        elif parts[0] == "blocks":
            out[f"{prefix}blocks.{parts[1]}.{inv_block[parts[2]]}.{parts[3]}"] = t
        elif parts[0] == "norm":
            out[f"{prefix}merger.norm.{parts[1]}"] = t
        elif parts[0] == "merge":
            out[f"{prefix}merger.linear_fc{1 if parts[1] == '0' else 2}.{parts[2]}"] = t
        elif parts[0] == "deepstack_norm":
            out[f"{prefix}deepstack_merger_list.{parts[1]}.norm.{parts[2]}"] = t
        elif parts[0] == "deepstack_merge":
            out[f"{prefix}deepstack_merger_list.{parts[1]}.linear_fc{1 if parts[2] == '0' else 2}.{parts[3]}"] = t
        else:
            raise KeyError(f"no Qwen3-VL name for '{k}'")
    return out


def hf_config_dict(cfg: MoTConfig, token_ids: Optional[Dict[str, int]] = None) -> Dict[str, object]:
    """`config.json` of a Qwen3-VL checkpoint with this model's shapes. `token_ids` names the ids of
    image_token_id / video_token_id / vision_start_token_id / vision_end_token_id in the tokenizer in use."""
    text = dict(model_type="qwen3_vl_text", vocab_size=cfg.vocab_size, hidden_size=cfg.d_model, intermediate_size=cfg.ffn_dim,
                num_hidden_layers=cfg.n_layers, num_attention_heads=cfg.n_heads, num_key_value_heads=cfg.n_kv_heads,
                head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_eps, hidden_act="silu", attention_bias=False,
                max_position_embeddings=262144, tie_word_embeddings=False,
                rope_parameters={"rope_type": "default", "rope_theta": float(cfg.rope_theta),
                                 "mrope_section": list(cfg.mrope_section), "mrope_interleaved": True})
    vision = dict(model_type="qwen3_vl", depth=cfg.vit_depth, hidden_size=cfg.vit_hidden, intermediate_size=cfg.vit_ffn or 4 * cfg.vit_hidden,
                  num_heads=cfg.vit_heads, patch_size=cfg.vit_patch, temporal_patch_size=cfg.vit_temporal_patch,
                  spatial_merge_size=cfg.vit_spatial_merge, out_hidden_size=cfg.d_model, in_channels=3,
                  num_position_embeddings=cfg.vit_pos_side ** 2, deepstack_visual_indexes=list(cfg.vit_deepstack),
                  hidden_act="gelu_pytorch_tanh")
    doc: Dict[str, object] = dict(model_type="qwen3_vl", architectures=["Qwen3VLForConditionalGeneration"], text_config=text,
                                  vision_config=vision, tie_word_embeddings=False)
    doc.update(token_ids or {})
    return doc


def load_vision_weights(vit, state: Mapping[str, torch.Tensor], strict: bool = True) -> None:
    vit.load_state_dict(vision_state_from_hf(state), strict=strict)


def load_checkpoint_dir(model, vit, model_dir, strict: bool = True) -> None:
    """Reads a Qwen3-VL checkpoint directory (safetensors shards, with or without an index) through the
    package's reader and fills the AR tower and, when given, the vision encoder."""
    from . import safetensors_io as sio

    state: Dict[str, torch.Tensor] = {}
    for name, path in sio.tensor_files(model_dir).items():
        state[name] = sio.open_reader(path).get(name)
    load_text_weights(model, state, strict)
    if vit is not None:
        load_vision_weights(vit, state, strict)


def hf_image_patches(video: torch.Tensor, patch: int, temporal_patch: int, merge: int) -> Optional[torch.Tensor]:
    """video [T, 3, H, W] -> the `pixel_values` layout of the Qwen3-VL processor: one row per patch, rows in the
    order (t, block row, block col, row in block, col in block), each row (C, temporal patch, patch, patch) flattened."""
    t_in, c, hh, ww = video.shape
    if t_in % temporal_patch:
        video = torch.cat([video, video[-1:].expand(temporal_patch - t_in % temporal_patch, -1, -1, -1)])
    t = video.shape[0] // temporal_patch
    gh, gw = hh // patch, ww // patch
    x = video.view(t, temporal_patch, c, gh // merge, merge, patch, gw // merge, merge, patch)
    return x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(t * gh * gw, c * temporal_patch * patch * patch)


def frames_from_hf_patches(pixels: torch.Tensor, grid_thw, patch: int, temporal_patch: int, merge: int) -> torch.Tensor:
    """Inverse of `hf_image_patches` for one image / clip: processor rows [t * gh * gw, C * tp * p * p] with their
    grid (t, gh, gw) -> frames [t * tp, 3, gh * p, gw * p]."""
    t, gh, gw = (int(v) for v in grid_thw)
    x = pixels.reshape(t, gh // merge, gw // merge, merge, merge, 3, temporal_patch, patch, patch)
    x = x.permute(0, 6, 5, 1, 3, 7, 2, 4, 8)
    return x.reshape(t * temporal_patch, 3, gh * patch, gw * patch)

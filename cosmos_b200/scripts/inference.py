"""Unified inference entry point, with the reference CLI's flags and output layout:

    python|torchrun -m cosmos_b200.scripts.inference -i spec.json(l) -o out_dir \
        --checkpoint-path Cosmos3-Nano --parallelism-preset=latency [--dp-shard-size N]
        [--dp-replicate-size N] [--cp-size N] [--cfgp-size N] [--seed N] [--no-guardrails]
        [--benchmark] [--video-save-quality 8] [--image_size 480]

(reference flags: cookbooks/cosmos3/generator/audiovisual/README.md:58-64, transfer/README.md:51,
evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb:643-649, reasoner/README.md:41-50,
action/run_fd_with_cosmos_framework.ipynb:652-653). Outputs, one directory per sample `name`:
`vision.mp4` (or `vision.png` for images), `reasoner_text.txt`, `sample_outputs.json`, and
`<out>/benchmark.json` with an `"average"` object when `--benchmark` is given.
Rendezvous uses MASTER_ADDR / MASTER_PORT / RANK / WORLD_SIZE / LOCAL_RANK.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

from ..config import DecodingConfig, ParallelConfig, SamplingConfig, get_model_config, resolve_size
from ..io import media
from ..io.spec import InferenceSpec, SpecError, load_specs


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="cosmos_b200.scripts.inference", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-i", "--input", required=True, help="input spec: .json (one sample) or .jsonl (one per line)")
    ap.add_argument("-o", "--output", required=True, help="output root; one sub-directory per sample name")
    ap.add_argument("--checkpoint-path", default="Cosmos3-Nano", help="model name (resolved under nvidia/) or path")
    ap.add_argument("--parallelism-preset", choices=["latency", "throughput"], default=None)
    ap.add_argument("--dp-shard-size", type=int, default=None)
    ap.add_argument("--dp-replicate-size", type=int, default=None)
    ap.add_argument("--cp-size", type=int, default=None)
    ap.add_argument("--cfgp-size", type=int, default=None)
    ap.add_argument("--tp-size", "--tensor-parallel-size", dest="tp_size", type=int, default=None)
    ap.add_argument("--cp-mode", choices=["ulysses", "ring"], default="ulysses")
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--no-guardrails", action="store_true")
    ap.add_argument("--benchmark", action="store_true")
    ap.add_argument("--video-save-quality", type=int, default=8)
    ap.add_argument("--image_size", "--image-size", dest="image_size", type=int, default=None)
    ap.add_argument("--enable-layerwise-offload", action="store_true",
                    help="accepted for compatibility; a no-op on 180 GB GPUs")
    ap.add_argument("--dtype", default=None, choices=["bf16", "fp32"])
    ap.add_argument("--device", default=None, help="cuda (default when available) or cpu")
    return ap


def resolve_parallelism(args, world: int, n_kv_heads: int, use_cfg: bool) -> ParallelConfig:
    """Explicit degrees win over the preset; unspecified degrees default to 1, and with only a
    preset the whole world is laid out by it. The product must equal the world size."""
    from ..config import preset_parallelism

    explicit = {k: getattr(args, k) for k in ("dp_shard_size", "dp_replicate_size", "cp_size", "cfgp_size", "tp_size")}
    if any(v is not None for v in explicit.values()):
        pc = ParallelConfig(dp_shard=explicit["dp_shard_size"] or 1, dp_replicate=explicit["dp_replicate_size"] or 1,
                            cp=explicit["cp_size"] or 1, cfgp=explicit["cfgp_size"] or 1, tp=explicit["tp_size"] or 1,
                            cp_mode=args.cp_mode)
        if pc.world != world and args.parallelism_preset == "throughput" and world % pc.world == 0:
            pc.dp_replicate *= world // pc.world
    else:
        pc = preset_parallelism(args.parallelism_preset or "latency", world, use_cfg=use_cfg, n_kv_heads=n_kv_heads)
    pc.validate(world)
    return pc


def _sampling_from_spec(s: InferenceSpec) -> SamplingConfig:
    return SamplingConfig(num_steps=s.num_steps, guidance=s.guidance, shift=s.shift, sigma_max=s.sigma_max,
                          guidance_interval=tuple(s.guidance_interval), normalize_cfg=s.normalize_cfg,
                          control_guidance=s.control_guidance, scheduler=s.scheduler, seed=s.seed)


def _size_for(spec: InferenceSpec):
    if spec.model_mode in ("forward_dynamics", "inverse_dynamics", "policy") and spec.image_size:
        return resolve_size(str(spec.image_size), spec.aspect_ratio)
    return resolve_size(spec.resolution, spec.aspect_ratio)


EDGE_PRESETS = {"very_low": (20, 50), "low": (50, 100), "medium": (100, 200), "high": (200, 300), "very_high": (300, 400)}
BLUR_PRESETS = {"very_low": 5, "low": 11, "medium": 21, "high": 31, "very_high": 41}


def _control_frames(spec: InferenceSpec, kind: str, ctrl: Dict, width: int, height: int) -> np.ndarray:
    """Frames [T, H, W, 3] of the control clip. `control_path` names a ready-made map; when that file is absent and the
    spec has an input video, edge and blur maps are computed from it (Canny thresholds / Gaussian kernel chosen by
    `preset_edge_threshold` / `preset_blur_strength`); depth, seg and wsm maps need their file."""
    path = spec.resolve(ctrl["control_path"]) if ctrl.get("control_path") else None
    if path is not None and Path(path).exists():
        frames, _ = media.read_video(path) if str(path).lower().endswith((".mp4", ".mov", ".mkv", ".webm", ".avi")) \
            else (media.read_image(path)[None], None)
        return np.asarray(frames)
    if kind not in ("edge", "blur") or not spec.vision_path:
        raise FileNotFoundError(f"control clip {path} not found (only edge and blur maps can be derived from the input video)")
    import cv2
    src, _ = media.read_video(spec.resolve(spec.vision_path))
    out = []
    for f in np.asarray(src):
        if kind == "edge":
            lo, hi = EDGE_PRESETS.get(str(ctrl.get("preset_edge_threshold", "medium")), EDGE_PRESETS["medium"])
            e = cv2.Canny(cv2.cvtColor(f, cv2.COLOR_RGB2GRAY), lo, hi)
            out.append(np.repeat(e[..., None], 3, axis=-1))
        else:
            k = BLUR_PRESETS.get(str(ctrl.get("preset_blur_strength", "medium")), BLUR_PRESETS["medium"])
            out.append(cv2.GaussianBlur(f, (k, k), 0))
    return np.stack(out)


def run_generator_sample(pipe, spec: InferenceSpec, out_dir: Path, quality: int, is_writer: bool) -> Dict:
    from ..data.vfm.action.av_dataset import DOMAIN_ACTION_DIM

    width, height = _size_for(spec)
    sc = _sampling_from_spec(spec)
    kw = {}
    image = video = None
    if spec.model_mode in ("image2video", "forward_dynamics", "policy"):
        image = spec.resolve(spec.vision_path)
    elif spec.model_mode in ("video2video", "inverse_dynamics") and spec.vision_path:
        video = spec.resolve(spec.vision_path)
        if spec.condition_frame_indexes_vision:
            kw["condition_frame_indexes"] = spec.condition_frame_indexes_vision
        elif spec.model_mode == "inverse_dynamics":
            kw["condition_frame_indexes"] = list(range((spec.num_frames - 1) // 4 + 1))
    if spec.is_transfer:
        # the control clip (edge / blur / depth / seg / wsm map) runs as a second, clean vision stream at the target's
        # positions; `control_guidance` and the hint's `control_weight` weigh its guidance branch
        kind, ctrl = next(iter(spec.controls.items()))
        kw["control_video"] = _control_frames(spec, kind, ctrl, width, height)
        kw["control_weight"] = float(ctrl.get("control_weight", 1.0))
        if video is not None and not spec.condition_frame_indexes_vision:
            n_first = spec.num_first_chunk_conditional_frames or 0
            if n_first:
                kw["condition_frame_indexes"] = list(range(1 + (n_first - 1) // pipe.cfg.vae_t_compress))
            else:
                video = None   # the input clip only served to derive the control map
    if spec.model_mode in ("forward_dynamics", "inverse_dynamics", "policy"):
        dom = spec.domain_name
        adim = spec.raw_action_dim or DOMAIN_ACTION_DIM.get(dom, 9)
        kw["domain"] = list(pipe.cfg.action_domains).index(dom)
        kw["action_dim"] = adim
        if spec.model_mode == "forward_dynamics":
            act = np.asarray(json.loads(spec.resolve(spec.action_path).read_text()), dtype=np.float32)
            kw["action"] = act[:spec.action_chunk_size]
        else:
            kw["n_action"] = spec.action_chunk_size
            kw["denoise_action"] = True
    if spec.negative_metadata_mode == "same":
        kw["negative_metadata_same"] = True
    negative = spec.negative_prompt_text((width, height)) or None
    t0 = time.perf_counter()
    per_chunk = spec.num_video_frames_per_chunk
    if per_chunk and spec.num_frames > per_chunk and image is None:
        # long clip: generated chunk by chunk, each chunk conditioned on the tail of the previous one
        kw.pop("condition_frame_indexes", None)
        out = pipe.generate_chunked(prompt=spec.prompt_text(), negative_prompt=negative,
                                    video=video, num_frames=spec.num_frames, height=height, width=width,
                                    fps=spec.fps, frames_per_chunk=per_chunk,
                                    num_conditional_frames=spec.num_conditional_frames or 1,
                                    num_first_chunk_conditional_frames=spec.num_first_chunk_conditional_frames or 0,
                                    sampling=sc, num_inference_steps=spec.num_steps, guidance_scale=spec.guidance,
                                    enable_sound=spec.enable_sound, **kw)
    else:
        out = pipe(prompt=spec.prompt_text(), negative_prompt=negative, image=image,
                   video=video, num_frames=spec.num_frames, height=height, width=width, fps=spec.fps,
                   num_inference_steps=spec.num_steps, guidance_scale=spec.guidance, enable_sound=spec.enable_sound,
                   sampling=sc, output_type="np", **kw)
    gen_s = time.perf_counter() - t0
    rec = {"name": spec.name, "model_mode": spec.model_mode, "generation_time_s": gen_s, **out.timings}
    if is_writer:
        out_dir.mkdir(parents=True, exist_ok=True)
        if spec.num_frames == 1:
            media.write_image(out_dir / "vision.png", out.video[0])
        else:
            rec["codec"] = media.write_video(out_dir / "vision.mp4", out.video, spec.fps, quality, out.sound,
                                             pipe.sound_tokenizer.config.sampling_rate)
        outputs = [{"content": {}}]
        if out.action is not None:
            outputs[0]["content"]["action"] = np.asarray(out.action).tolist()
        (out_dir / "sample_outputs.json").write_text(json.dumps({"name": spec.name, "outputs": outputs,
                                                                 "spec": spec.to_dict()}))
    return rec


def _reasoner_prompt(tokenizer, vit, cfg, spec: InferenceSpec, device):
    """Token ids of the chat prompt and, for a prompt with media, the vision rows, grid, pad id and DeepStack features."""
    from ..models.vae import CausalVideoVAE

    content, vision_embeds, grids, n_vis, deep = [], None, [], [], None
    if spec.vision_path:
        # clips are sampled at 2 frames per second (at most 32 frames), as the serving path does by default
        frames, times, _ = media.sample_video(spec.resolve(spec.vision_path), fps=2.0, limit=32)
        from ..serve.server import smart_resize
        unit = cfg.vit_patch * cfg.vit_spatial_merge
        most = 12845056 if frames.shape[0] == 1 else min(12845056, 25165824 // frames.shape[0])
        h, w = smart_resize(frames.shape[1], frames.shape[2], unit, min(3136, most), most)
        from PIL import Image
        fr = np.stack([np.asarray(Image.fromarray(f).resize((w, h))) for f in frames])
        vid = CausalVideoVAE.from_uint8(torch.from_numpy(fr)[None])[0].permute(1, 0, 2, 3).to(device)
        with torch.no_grad():
            vision_embeds, grid, deep = vit(vid, return_deepstack=True)
        is_video = frames.shape[0] > 1
        if is_video:   # one time-stamped vision segment (and rotary grid) per temporal group
            from ..utils.tokenizer import video_layout
            grids, n_vis = [(1, grid[1], grid[2])] * grid[0], [video_layout(grid, times, cfg.vit_temporal_patch)]
        else:
            grids, n_vis = [grid], [grid[0] * grid[1] * grid[2]]
        content.append({"type": "video_url" if is_video else "image_url"})
    content.append({"type": "text", "text": spec.prompt_text()})
    ids = tokenizer.apply_chat_template([{"role": "user", "content": content}], True, n_vis)
    pad_id = tokenizer.video_pad_id if (spec.vision_path and is_video) else tokenizer.image_pad_id
    return ids, vision_embeds, grids, pad_id, deep


def run_reasoner_batch(pipe, vit, specs: List[InferenceSpec], out_root: Path, is_writer: bool, device,
                       max_num_seqs: int = 32) -> List[Dict]:
    """All reasoner samples of a spec file through the continuous-batching engine (`serve/engine.py`): they
    share decode steps (one CUDA graph per step on a GPU), each with its own sampling parameters."""
    from ..models.reasoner import ReasonerEngine
    from ..serve.engine import BatchEngine

    tok, ref = pipe.tokenizer, ReasonerEngine(pipe.transformer, vit)
    prompts = [_reasoner_prompt(tok, vit, pipe.cfg, s, device) for s in specs]
    longest = max(len(p[0]) + s.max_new_tokens for p, s in zip(prompts, specs))
    eng = BatchEngine(pipe.transformer, max_batch=min(max_num_seqs, len(specs)), max_len=longest + 16)
    t0 = time.perf_counter()
    reqs = []
    for s, (ids, ve, grids, pad_id, deep) in zip(specs, prompts):
        kw = {}
        if ve is not None:
            ids_t = torch.tensor([ids], dtype=torch.long, device=device)
            vmask = ids_t == pad_id
            x = ref.embed(ids_t.clamp(max=pipe.cfg.vocab_size - 1), ve, vmask)
            kw = dict(embeds=x[0], positions=ref.positions(ids_t, vmask, grids), vision_mask=vmask[0], deepstack=deep)
        reqs.append(eng.submit(ids, s.max_new_tokens, (tok.eos_id, tok.eot_id),
                               temperature=s.temperature if s.do_sample else 0.0, top_k=s.top_k, top_p=s.top_p,
                               presence_penalty=s.presence_penalty, repetition_penalty=s.repetition_penalty, **kw))
    eng.run_until_done()
    if device.type == "cuda":
        torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    records = []
    for s, r in zip(specs, reqs):
        if is_writer:
            d = out_root / s.name
            d.mkdir(parents=True, exist_ok=True)
            (d / "reasoner_text.txt").write_text(tok.decode(r.out))
        dt = max(r.t_done - r.t_submit, 1e-9)
        records.append({"name": s.name, "model_mode": "reasoner", "generation_time_s": dt,
                        "tokens_per_s": len(r.out) / dt, "prompt_tokens": len(r.ids), "completion_tokens": len(r.out),
                        "batch_wall_s": wall, "batch_tokens_per_s": sum(len(q.out) for q in reqs) / max(wall, 1e-9)})
    return records


def run_reasoner_sample(engine, tokenizer, vit, spec: InferenceSpec, out_dir: Path, is_writer: bool, device) -> Dict:
    from ..models.vae import CausalVideoVAE

    messages_content = []
    vision_embeds, grids, n_vis, deep = None, [], [], None
    if spec.vision_path:
        # clips are sampled at 2 frames per second (at most 32 frames), as the serving path does by default
        frames, times, _ = media.sample_video(spec.resolve(spec.vision_path), fps=2.0, limit=32)
        unit = engine.cfg.vit_patch * engine.cfg.vit_spatial_merge
        h = max(unit, frames.shape[1] // unit * unit)
        w = max(unit, frames.shape[2] // unit * unit)
        h, w = min(h, 14 * unit), min(w, 14 * unit)
        from PIL import Image
        fr = np.stack([np.asarray(Image.fromarray(f).resize((w, h))) for f in frames])
        vid = CausalVideoVAE.from_uint8(torch.from_numpy(fr)[None])[0].permute(1, 0, 2, 3).to(device)
        with torch.no_grad():
            vision_embeds, grid, deep = vit(vid, return_deepstack=True)
        grids, n_vis = [grid], [grid[0] * grid[1] * grid[2]]
        messages_content.append({"type": "image_url" if frames.shape[0] == 1 else "video_url"})
    messages_content.append({"type": "text", "text": spec.prompt_text()})
    ids = tokenizer.apply_chat_template([{"role": "user", "content": messages_content}], True, n_vis)
    dc = DecodingConfig(max_new_tokens=spec.max_new_tokens, do_sample=spec.do_sample, temperature=spec.temperature,
                        top_p=spec.top_p, top_k=spec.top_k, repetition_penalty=spec.repetition_penalty,
                        presence_penalty=spec.presence_penalty, seed=spec.seed)
    pad_id = tokenizer.video_pad_id if (grids and grids[0][0] > 1) else tokenizer.image_pad_id
    t0 = time.perf_counter()
    out_ids, usage = engine.generate(ids, dc, eos_ids=(tokenizer.eos_id, tokenizer.eot_id),
                                     vision_embeds=vision_embeds, vision_token_id=pad_id if grids else None,
                                     grids=grids, deepstack=deep)
    dt = time.perf_counter() - t0
    text = tokenizer.decode(out_ids)
    if is_writer:
        out_dir.mkdir(parents=True, exist_ok=True)
        (out_dir / "reasoner_text.txt").write_text(text)
    return {"name": spec.name, "model_mode": "reasoner", "generation_time_s": dt,
            "tokens_per_s": usage["completion_tokens"] / max(dt, 1e-9), **usage}


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    overrides = {"seed": args.seed, "image_size": args.image_size}
    try:
        specs = load_specs(args.input, overrides)
    except SpecError as e:
        print(f"spec error: {e}", file=sys.stderr)
        return 2
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and args.device != "cpu"
    if use_cuda:
        torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    dtype = torch.bfloat16 if (args.dtype or ("bf16" if use_cuda else "fp32")) == "bf16" else torch.float32
    cfg = get_model_config(args.checkpoint_path) if not Path(args.checkpoint_path).is_dir() else None
    from ..parallel.runtime import build_engine_for_mesh, init_distributed

    use_cfg = any(s.is_generator and s.guidance != 1.0 for s in specs)
    n_kv = cfg.n_kv_heads if cfg is not None else 8
    try:
        pc = resolve_parallelism(args, world, n_kv, use_cfg)
    except ValueError as e:
        print(f"parallelism error: {e}", file=sys.stderr)
        return 2
    mesh = init_distributed(world, rank, local_rank, pc=pc, backend=None if use_cuda else "gloo")
    out_root = Path(args.output)
    if rank == 0:
        out_root.mkdir(parents=True, exist_ok=True)

    from ..pipeline import Cosmos3OmniPipeline

    pipe = Cosmos3OmniPipeline.from_pretrained(args.checkpoint_path, torch_dtype=dtype,
                                               device_map=str(device) if use_cuda else None,
                                               enable_safety_checker=not args.no_guardrails)
    pipe.engine = build_engine_for_mesh(pipe.transformer, mesh)
    reasoner = vit = None
    # replicas (dp_replicate) take different samples; all other ranks of a replica work on the same one
    replica, n_rep = mesh.index("dp_replicate"), mesh.size("dp_replicate")
    is_writer = all(mesh.index(a) == 0 for a in ("dp_shard", "cfgp", "cp", "tp"))
    records = []
    mine = [s for i, s in enumerate(specs) if i % n_rep == replica]
    batched = set()
    # several reasoner samples (or any on a GPU) go through the batching engine; seeds pinned per sample and
    # multi-rank layouts keep the per-sample path
    rs = [s for s in mine if s.model_mode == "reasoner"]
    if rs and world == 1 and (use_cuda or len(rs) > 1) and os.environ.get("COSMOS_REASONER_SINGLE") != "1":
        from ..models.vit import VisionEncoder
        vit = pipe.vision_encoder()
        for rec in run_reasoner_batch(pipe, vit, rs, out_root, is_writer, device):
            records.append(rec)
            if is_writer:
                print(json.dumps(rec), flush=True)
        batched = {s.name for s in rs}
    for i, spec in enumerate(specs):
        if i % n_rep != replica or spec.name in batched:
            continue
        out_dir = out_root / spec.name
        if spec.model_mode == "reasoner":
            if reasoner is None:
                from ..models.reasoner import ReasonerEngine
                from ..models.vit import VisionEncoder
                vit = pipe.vision_encoder()
                reasoner = ReasonerEngine(pipe.transformer, vit)
            rec = run_reasoner_sample(reasoner, pipe.tokenizer, vit, spec, out_dir, is_writer, device)
        else:
            for k in range(spec.num_outputs):
                sp = spec if spec.num_outputs == 1 else InferenceSpec(**{**spec.to_dict(), "seed": spec.seed + k,
                                                                         "name": f"{spec.name}_{k}"})
                sp.spec_dir = spec.spec_dir
                rec = run_generator_sample(pipe, sp, out_root / sp.name, args.video_save_quality, is_writer)
        records.append(rec)
        if is_writer:
            print(json.dumps(rec), flush=True)
    if args.benchmark and is_writer:
        avg = {}
        for key in ("generation_time_s", "sample_s", "decode_s", "prepare_s", "tokens_per_s"):
            vals = [r[key] for r in records if key in r]
            if vals:
                avg[key] = sum(vals) / len(vals)
        name = "benchmark.json" if n_rep == 1 else f"benchmark_replica{replica}.json"
        (out_root / name).write_text(json.dumps({"average": avg, "samples": records, "parallelism": mesh.describe(),
                                                 "world_size": world}, indent=1))
    if world > 1:
        from ..parallel.runtime import finish
        finish(hard=(__name__ == "__main__"))
    return 0


if __name__ == "__main__":
    sys.exit(main())

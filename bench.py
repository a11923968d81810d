"""Benchmarks of the metrics named for Cosmos3 on N GPUs of one node, one JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|library|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Headline (`value`): latency of one guided DiT denoise step of Cosmos3-Nano text-to-video at 720p
(121 frames -> 31x90x160x16 latent -> 111,600 video tokens, 512 text tokens per branch, cond + uncond
branches, CFG combine and Euler update). Layout per N: 1 = both branches as one batch on one GPU;
2 = CFG-parallel (one branch per GPU); 4 and 8 = CFG-parallel x Ulysses context-parallel (N/2 ranks per
branch); `--tp-size / --cp-size / --cfgp-size / --cp-mode` pick another layout (e.g. `--model Cosmos3-Super
--tp-size 8`). Total work is fixed ("strong" scaling). Timing: W untimed warm-up steps, then exactly K steps
between CUDA events bracketed by barrier + synchronize, max over ranks. Each step streams far more than the
126 MB L2 (16 GB of weights, GBs of activations), so no explicit L2 flush is needed between steps. SM clocks
and throttle reasons are sampled with nvidia-smi during every timed region. The `e2e` figure runs the same
steps through the public `Cosmos3OmniPipeline.step_from_host` call, which copies the step's latents from
pinned host memory to the GPU and the result back.

The same line also carries the other named metrics, each device-timed (max over ranks) with its own clock
sample, under `extra`:
  * `s_per_video`: measured prompt prefill (AR tower, both branches) + 35 x the measured step + measured
    tokenizer decode of the 31x90x160 latent to 121x720x1280x3 uint8;
  * `decode_tok_s`: Reasoner greedy decode, tensor parallel over the N GPUs, batch 32, 8448-token contexts
    in a paged KV cache, 256 new tokens, one CUDA graph per step;
  * `train_tok_s`: one FSDP (x context-parallel 2 from N >= 2) post-training step of the DM tower on
    16x16x44x80 latents with 256 text ids, activation checkpointing, AdamW, grad-clip 1.0.
A phase that fails or runs out of its time budget is reported as an error string and does not affect the
headline. `--no-extras` skips them.

`--impl library`: the same model, layout and sampler with every op on PyTorch's library kernels (cuBLAS,
fused SDPA, eager element-wise) and NCCL collectives instead of this package's kernels: the A/B arm.
`--impl reference`: the reference repository ships no source code to install or run (documentation and
notebooks only), so that arm prints an `unavailable` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import traceback

# published per-step latency derived from the reference's Nano T2V 720p table
# (inference_benchmarks.md:63, PyTorch engine, seconds per 35-step generation)
PUBLISHED_S_PER_VIDEO = {1: 114.85, 4: 39.75, 8: 26.27}
PUBLISHED_STEPS = 35
PUBLISHED_DECODE_TOK_S = 2701.08   # inference_benchmarks.md:525 (Nano, out 100, 1 FPS, c=256; a served instance)


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001 - nvidia-smi missing: report no clocks
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.strip().split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); power.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference repository contains no installable source (documentation, notebooks and one "
                      "122-line ffmpeg helper; no pyproject/setup.py), so pip cannot build it and there is no "
                      "stock code path to run"}))
    return 0


def _peaks():
    p = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(p))
        return d["bf16_tflops_sustained"], d["hbm_gbs"], "measured"
    except Exception:  # noqa: BLE001
        return 1400.0, 6650.0, "fallback"


class Ctx:
    """What every phase needs: torch, the ranks, a barrier + synchronize, and a max over ranks."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = torch.device("cuda", self.local_rank)
        self.library = args.impl == "library"

    def sync(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, *vals):
        t = self.torch.tensor(list(vals), device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def sampler(self):
        return ClockSampler(self.local_rank).start() if self.rank == 0 else None

    def free(self):
        import gc
        gc.collect()
        self.torch.cuda.empty_cache()


# ----------------------------------------------------------------------------- phase 1: guided DiT step
def phase_dit(c: Ctx, rec: dict):
    torch, args = c.torch, c.args
    from cosmos_b200 import ops
    from cosmos_b200.config import SamplingConfig, latent_shape, resolve_size
    from cosmos_b200.parallel.runtime import build_engine_for_mesh, init_distributed
    from cosmos_b200.pipeline import Cosmos3OmniPipeline

    pc = None
    if args.tp_size or args.cp_size or args.cfgp_size:
        from cosmos_b200.config import ParallelConfig
        pc = ParallelConfig(tp=max(1, args.tp_size), cp=max(1, args.cp_size), cfgp=max(1, args.cfgp_size),
                            cp_mode=args.cp_mode)
        pc.validate(c.world)
    mesh = init_distributed(c.world, c.rank, c.local_rank, preset="latency", pc=pc)
    overrides = {"max_text_len": args.text_len}
    if args.layers:
        overrides["n_layers"] = args.layers
    full_cfg = None
    if mesh.size("tp") > 1:
        # every rank builds only its slice of the block weights (1 / tp of the heads and FFN units)
        from cosmos_b200.config import get_model_config
        from cosmos_b200.parallel.tp import tp_local_config
        full_cfg = get_model_config(args.model, **overrides)
        loc = tp_local_config(full_cfg, mesh.size("tp"))
        overrides.update(n_heads=loc.n_heads, n_kv_heads=loc.n_kv_heads, ffn_dim=loc.ffn_dim)
    pipe = Cosmos3OmniPipeline.from_pretrained(args.model, torch_dtype=torch.bfloat16,
                                               device_map=f"cuda:{c.local_rank}", enable_safety_checker=False,
                                               config_overrides=overrides, engine_kwargs=None,
                                               layer_seed=(1 + mesh.index("tp")) if full_cfg is not None else None)
    pipe.engine = build_engine_for_mesh(pipe.transformer, mesh, fused=not c.library, full_cfg=full_cfg)
    cfg = pipe.cfg
    weight_gb = sum(p.numel() * p.element_size() for p in pipe.transformer.parameters()) / 2 ** 30
    width, height = resolve_size(args.resolution)
    grid = latent_shape(cfg, args.frames, width, height)
    n_tokens = (grid[0] // cfg.patch_t) * (grid[1] // cfg.patch_hw) * (grid[2] // cfg.patch_hw)
    dev = c.dev

    # synthetic inputs: random prompt ids for both branches, N(0,1) latent
    g = torch.Generator(device=dev).manual_seed(1234)
    ids_c = torch.randint(0, cfg.vocab_size, (1, args.text_len), generator=g, device=dev)
    ids_u = torch.randint(0, cfg.vocab_size, (1, args.text_len), generator=g, device=dev)
    total_steps = args.warmup + args.steps + 1 + args.e2e_steps + 1
    sc = SamplingConfig(num_steps=max(35, total_steps), guidance=args.guidance, shift=10.0, scheduler="euler", seed=0)
    st = pipe.engine.make_state(ids_c, ids_u, grid)   # warm-up of the prefill path
    c.sync()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    st = pipe.engine.make_state(ids_c, ids_u, grid)
    p1.record()
    c.sync()
    prefill_ms = p0.elapsed_time(p1)
    x = pipe.begin(st, sc)

    step_i = 0
    for _ in range(args.warmup):
        x = pipe.step(x, step_i); step_i += 1
    c.sync()
    ops.check_status()
    launches0 = ops.launch_count()
    sampler = c.sampler()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c.sync()
    torch.cuda.cudart().cudaProfilerStart()  # lets a profiler started with --profile-from-start off see only the timed steps
    e0.record()
    for _ in range(args.steps):
        x = pipe.step(x, step_i); step_i += 1
    e1.record()
    c.sync()
    torch.cuda.cudart().cudaProfilerStop()
    clocks = sampler.stop() if sampler else None
    launches = ops.launch_count() - launches0
    ms = e0.elapsed_time(e1) / args.steps
    ops.check_status()

    # end-to-end through the public host API (pinned host -> device -> step -> host)
    host_in = torch.empty(x.shape, dtype=torch.float32).pin_memory()
    host_out = torch.empty(x.shape, dtype=torch.float32).pin_memory()
    host_in.copy_(x)
    pipe.step_from_host(host_in, step_i, host_out); step_i += 1   # warm-up of the host path
    c.sync()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.e2e_steps):
        pipe.step_from_host(host_in, step_i, host_out); step_i += 1
        host_in, host_out = host_out, host_in
    e3.record()
    c.sync()
    e2e_ms = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3) / max(1, args.e2e_steps)
    ops.check_status()
    finite = bool(torch.isfinite(host_in).all())
    ms, e2e_ms, prefill_ms = c.max_over_ranks(ms, e2e_ms, prefill_ms)

    pub = PUBLISHED_S_PER_VIDEO.get(c.world) if args.model == "Cosmos3-Nano" else None   # the table is Nano's
    if args.model == "Cosmos3-Super" and c.world == 8:
        pub = 65.91   # Super I2V 720p on 8 GPUs, PyTorch engine (inference_benchmarks.md:193)
    base_ms = None if pub is None else pub * 1e3 / PUBLISHED_STEPS
    rec.update({
        "metric": f"dit_step_ms ({args.model} T2V {args.resolution}p, one guided denoise step: cond+uncond forward, CFG, Euler)",
        "value": round(ms, 3), "unit": "ms", "n_gpus": c.world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None if base_ms is None else round(ms / base_ms, 4),
        "dtype": "bf16", "data": "synthetic (random token ids, N(0,1) latent, random-init weights)",
        "impl": args.impl,
        "config": {"model": cfg.name + (" (layer override: INVALID as headline)" if args.layers else ""),
                   "global_batch": 1, "seq_len": n_tokens + args.text_len, "video_tokens": n_tokens,
                   "text_tokens": args.text_len, "frames": args.frames, "resolution": f"{width}x{height}",
                   "layers": cfg.n_layers, "cfg_scale": args.guidance, "parallelism": mesh.describe(),
                   "transformer_weights_gib_per_gpu": round(weight_gb, 2),
                   "l2": "inputs larger than L2 (16 GB weights + GBs of activations per step)",
                   "baseline_note": "published number is for the reference's own 189-frame model, whose "
                                    "compute per token is far below these dense stand-in shapes"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_ms, 3), "unit": "ms",
                "h2d_bytes_per_step": int(host_in.numel() * 4), "d2h_bytes_per_step": int(host_out.numel() * 4)},
        "gpu_launches": int(launches),
        "finite_output": finite,
    })
    extra = rec.setdefault("extra", {})
    extra["prefill_ms"] = round(prefill_ms, 2)
    if not args.no_extras:
        # tokenizer decode of the final latent to 121 x 720 x 1280 x 3 uint8 (rank 0's GPU does the work; every rank
        # takes part in the gather of the context-parallel shards)
        try:
            frames = pipe.decode(x, st)[0]   # warm-up (weight repacking, workspaces)
            c.sync()
            smp = c.sampler()
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            d0.record()
            frames = pipe.decode(x, st)[0]
            d1.record()
            c.sync()
            dec_ms = max(d0.elapsed_time(d1), (time.perf_counter() - t0) * 1e3)   # includes the copy of the frames to the host
            (dec_ms,) = c.max_over_ranks(dec_ms)
            extra["vae_decode_ms"] = round(dec_ms, 2)
            extra["vae_decode_frames"] = list(frames.shape)
            extra["vae_decode_clocks"] = smp.stop() if smp else None
            s_video = (prefill_ms + PUBLISHED_STEPS * ms + dec_ms) / 1e3
            extra["s_per_video"] = {"value": round(s_video, 2), "unit": "s",
                                    "what": "measured prefill + 35 x measured guided step + measured tokenizer decode",
                                    "vs_published": None if pub is None else round(s_video / pub, 3)}
        except Exception as e:  # noqa: BLE001 - the headline stands without it
            extra["s_per_video"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    rec["s_per_video_35_steps"] = round(ms * 35 / 1e3, 2)
    del pipe, st, x
    c.free()
    return mesh


# ----------------------------------------------------------------------------- phase 2: Reasoner decode
def phase_decode(c: Ctx, rec: dict):
    torch, dist = c.torch, c.dist
    from cosmos_b200 import ops
    from cosmos_b200.config import get_model_config
    from cosmos_b200.serve.decoder import TPDecoder

    a = c.args
    cfg = get_model_config("Cosmos3-Nano", **({"n_layers": a.layers} if a.layers else {}))
    batch, prompt, new = 32, 8192 + 256, 256
    warm = 8
    dec = TPDecoder(cfg, c.world, c.rank, dist.group.WORLD if c.world > 1 else None, c.dev, max_batch=batch,
                    max_len=prompt + new + warm + 8, fused=not c.library)
    dec.prefill_synthetic(batch, prompt, new + warm + 8)
    dec.capture(warmup=warm - 1)
    c.sync()
    smp = c.sampler()
    l0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(new):
        dec.step()
    e1.record()
    c.sync()
    ops.check_status()
    clocks = smp.stop() if smp else None
    (ms,) = c.max_over_ranks(e0.elapsed_time(e1))
    toks = batch * new
    kv_bytes = 2 * cfg.n_layers * batch * (prompt + new / 2) * (cfg.n_kv_heads // c.world) * cfg.head_dim * 2
    w_bytes = (cfg.tower_params() // c.world + (cfg.vocab_size // c.world) * cfg.d_model) * 2
    _, hbm, src = _peaks()
    floor_ms = (kv_bytes + w_bytes) / (hbm * 1e9) * 1e3
    rec["extra"]["decode_tok_s"] = {
        "value": round(toks / ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(ms / new, 4),
        "config": {"model": cfg.name, "tp": c.world, "batch": batch, "context": prompt, "new_tokens": new,
                   "paged_kv": True, "cuda_graph": True, "fused_allreduce": not c.library and c.world > 1,
                   "prefill": "synthetic K/V (N(0,1)) written into the pages"},
        f"fraction_of_{src}_hbm_floor": round(floor_ms / (ms / new), 3),
        "vs_published_served_c256": round(toks / ms * 1e3 / PUBLISHED_DECODE_TOK_S, 3),
        "clocks": clocks}
    del dec
    c.free()


# ----------------------------------------------------------------------------- phase 3: FSDP x CP training step
def phase_train(c: Ctx, rec: dict):
    torch, dist = c.torch, c.dist
    from cosmos_b200 import ops
    from cosmos_b200.config import ParallelConfig, get_model_config
    from cosmos_b200.models.mot import MoTModel
    from cosmos_b200.parallel.mesh import Mesh
    from cosmos_b200.train import TrainConfig, Trainer

    a = c.args
    cp = 2 if c.world >= 2 else 1
    dshard = c.world // cp
    mesh = Mesh(ParallelConfig(dp_shard=dshard, cp=cp), c.world, c.rank)
    cfg = get_model_config("Cosmos3-Nano", **({"n_layers": a.layers} if a.layers else {}))
    if c.library:
        os.environ["COSMOS_TRAIN_LIBRARY_BACKWARD"] = "1"
    model = MoTModel(cfg, dtype=torch.bfloat16, device=c.dev, pad_to=128 * dshard * cp)
    model.init_weights(seed=0)
    tr = Trainer(model, mesh, TrainConfig(lr=1e-4, max_grad_norm=1.0, checkpoint_blocks=True, fused=not c.library))
    ch, t, h, w = 16, 16, 44, 80
    text_len = 256
    data_rank = mesh.index("dp_shard")
    g = torch.Generator(device=c.dev).manual_seed(1000 + data_rank)
    tokens_per_step = ((t // cfg.patch_t) * (h // cfg.patch_hw) * (w // cfg.patch_hw) + text_len) * dshard

    def one_step():
        # inputs start in pinned host memory, as a data loader would hand them over
        lat_h = torch.randn(1, ch, t, h, w, dtype=torch.bfloat16).pin_memory()
        ids_h = torch.randint(0, cfg.vocab_size, (1, text_len)).pin_memory()
        if cp > 1:   # the ranks of one context-parallel group train on the same clip
            lat = lat_h.to(c.dev, non_blocking=True); ids = ids_h.to(c.dev, non_blocking=True)
            dist.broadcast(lat, src=mesh.group_ranks["cp"][0], group=mesh.group("cp"))
            dist.broadcast(ids, src=mesh.group_ranks["cp"][0], group=mesh.group("cp"))
        else:
            lat = lat_h.to(c.dev, non_blocking=True); ids = ids_h.to(c.dev, non_blocking=True)
        return tr.train_step(lat, ids, g)

    for _ in range(2):
        out = one_step()
    c.sync()
    ops.check_status()
    n_steps = 3
    smp = c.sampler()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_steps):
        out = one_step()
    e1.record()
    c.sync()
    ops.check_status()
    clocks = smp.stop() if smp else None
    (ms,) = c.max_over_ranks(e0.elapsed_time(e1) / n_steps)
    tf, _, src = _peaks()
    # 6 x params x tokens for the DM tower's linear layers (+ 2 x for the recomputed forward), attention 4 S^2 d per layer
    # forward (x 3.5 with backward and recomputation), per clip; clips per step = dshard
    s_tok = tokens_per_step // dshard
    flops = dshard * (8.0 * cfg.tower_params() * s_tok + 3.5 * 4.0 * s_tok * s_tok * cfg.q_dim * cfg.n_layers)
    floor_s = flops / (tf * 1e12 * c.world)
    rec["extra"]["train_tok_s"] = {
        "value": round(tokens_per_step / ms * 1e3, 1), "unit": "tokens/s", "step_ms": round(ms, 2),
        "loss": out.get("loss"), "grad_norm": out.get("grad_norm"),
        "config": {"model": cfg.name, "parallelism": mesh.describe(), "clips_per_step": dshard,
                   "tokens_per_clip": s_tok, "latent": [ch, t, h, w], "text_len": text_len,
                   "activation_checkpointing": True, "grad_clip": 1.0, "optimizer": "AdamW",
                   "fused_collectives": not c.library and c.world > 1},
        f"fraction_of_{src}_compute_floor": round(floor_s / (ms / 1e3), 3),
        "clocks": clocks}
    del tr, model
    c.free()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "library", "reference"])
    ap.add_argument("--model", default="Cosmos3-Nano")
    ap.add_argument("--frames", type=int, default=121)
    ap.add_argument("--resolution", default="720")
    ap.add_argument("--text-len", type=int, default=512)
    ap.add_argument("--guidance", type=float, default=7.0)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--tp-size", type=int, default=0, help="explicit layout instead of the latency preset: tensor parallel")
    ap.add_argument("--cp-size", type=int, default=0, help="explicit layout: context parallel (Ulysses; --cp-mode ring)")
    ap.add_argument("--cfgp-size", type=int, default=0, help="explicit layout: CFG parallel (1 or 2)")
    ap.add_argument("--cp-mode", default="ulysses", choices=["ulysses", "ring"])
    ap.add_argument("--no-extras", action="store_true", help="headline only (no s/video, decode, training phases)")
    ap.add_argument("--extras", default="video,decode,train", help="which extra phases to run")
    ap.add_argument("--extras-budget-s", type=float, default=330.0,
                    help="a phase is not started once the extras have used this much wall time")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from cosmos_b200 import ops

    c = Ctx(args)
    if c.world != args.gpus:
        if c.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
        args.gpus = c.world
    torch.cuda.set_device(c.local_rank)
    if not ops.load_extension():
        raise SystemExit("cosmos_b200 kernel library failed to load")
    if c.library:
        ops.set_backend("library")
    rec: dict = {}
    phase_dit(c, rec)
    t_extra = time.perf_counter()
    running = {"phase": None}

    def watchdog():
        # A phase that blocks (a rank that failed alone leaves the others inside a collective) must not cost the
        # headline: past the deadline rank 0 prints what it has and every rank leaves.
        deadline = args.extras_budget_s + 150.0
        while time.perf_counter() - t_extra < deadline:
            time.sleep(1.0)
            if running["phase"] == "done":
                return
        if c.rank == 0:
            if running["phase"]:
                rec.setdefault("extra", {})[running["phase"]] = {"error": "phase did not finish before the bench deadline"}
            print(json.dumps(rec), flush=True)
        sys.stdout.flush()
        os._exit(0)

    if not args.no_extras:
        threading.Thread(target=watchdog, daemon=True).start()
    if not args.no_extras and args.model == "Cosmos3-Nano":
        for name, fn in (("decode", phase_decode), ("train", phase_train)):
            if name not in args.extras.split(","):
                continue
            if c.library and name == "decode":
                rec["extra"]["decode_tok_s"] = {"skipped": "no library counterpart of the paged-KV decode step is wired into this arm"}
                continue
            # every rank takes the same decision (rank 0's clock) so that no rank enters a collective alone
            spent = c.max_over_ranks(time.perf_counter() - t_extra)[0]
            key = {"decode": "decode_tok_s", "train": "train_tok_s"}[name]
            if spent > args.extras_budget_s:
                rec["extra"][key] = {"skipped": f"extras time budget used up ({spent:.0f} s)"}
                continue
            running["phase"] = key
            try:
                fn(c, rec)
            except Exception as e:  # noqa: BLE001 - reported in the line; the headline stands
                rec["extra"][key] = {"error": f"{type(e).__name__}: {e}"[:400]}
                if c.rank == 0:
                    traceback.print_exc(file=sys.stderr)
                try:
                    torch.ops.cosmos_b200.status_word().zero_()
                except Exception:  # noqa: BLE001
                    pass
                c.free()
    running["phase"] = "done"
    if c.rank == 0:
        print(json.dumps(rec), flush=True)
    if c.world > 1:
        from cosmos_b200.parallel.runtime import finish
        finish(hard=(__name__ == "__main__"))
    return 0


if __name__ == "__main__":
    sys.exit(main())

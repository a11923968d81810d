"""Headline benchmark: latency of one guided DiT denoise step of Cosmos3-Nano text-to-video at
720p (121 frames -> 31x90x160x16 latent -> 111,600 video tokens, 512 text tokens per branch,
cond + uncond branches, CFG combine and Euler update), on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Layout per N: 1 = both branches as one batch on one GPU; 2 = CFG-parallel (one branch per GPU);
4 and 8 = CFG-parallel x Ulysses context-parallel (N/2 ranks per branch); `--tp-size / --cp-size / --cfgp-size /
--cp-mode` pick another layout (e.g. `--model Cosmos3-Super --tp-size 8`). Total work is fixed
("strong" scaling). Timing: W untimed warm-up steps, then exactly K steps between CUDA events
bracketed by barrier + synchronize, max over ranks. Each step streams far more than the 126 MB
L2 (16 GB of weights, GBs of activations), so no explicit L2 flush is needed between steps.
SM clocks and throttle reasons are sampled with nvidia-smi during the timed region.
The `e2e` figure runs the same steps through the public `Cosmos3OmniPipeline.step_from_host`
call, which copies the step's latents from pinned host memory to the GPU and the result back.

`--impl reference`: the reference repository ships no source code to install or run
(documentation and notebooks only), so that arm prints an `unavailable` line.
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

# published per-step latency derived from the reference's Nano T2V 720p table
# (inference_benchmarks.md:63, PyTorch engine, seconds per 35-step generation)
PUBLISHED_S_PER_VIDEO = {1: 114.85, 4: 39.75, 8: 26.27}
PUBLISHED_STEPS = 35


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
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
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from cosmos_b200 import ops
    from cosmos_b200.config import SamplingConfig, get_model_config, latent_shape, resolve_size
    from cosmos_b200.parallel.runtime import build_engine_for_mesh, init_distributed
    from cosmos_b200.pipeline import Cosmos3OmniPipeline

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pc = None
    if args.tp_size or args.cp_size or args.cfgp_size:
        from cosmos_b200.config import ParallelConfig
        pc = ParallelConfig(tp=max(1, args.tp_size), cp=max(1, args.cp_size), cfgp=max(1, args.cfgp_size), cp_mode=args.cp_mode)
        pc.validate(world)
    mesh = init_distributed(world, rank, local_rank, preset="latency", pc=pc)
    if not ops.load_extension():
        raise SystemExit("cosmos_b200 kernel library failed to load")

    overrides = {"max_text_len": args.text_len}
    if args.layers:
        overrides["n_layers"] = args.layers
    pipe = Cosmos3OmniPipeline.from_pretrained(args.model, torch_dtype=torch.bfloat16, device_map=f"cuda:{local_rank}",
                                               enable_safety_checker=False, config_overrides=overrides,
                                               engine_kwargs=None)
    pipe.engine = build_engine_for_mesh(pipe.transformer, mesh)
    cfg = pipe.cfg
    width, height = resolve_size(args.resolution)
    grid = latent_shape(cfg, args.frames, width, height)
    n_tokens = (grid[0] // cfg.patch_t) * (grid[1] // cfg.patch_hw) * (grid[2] // cfg.patch_hw)

    # synthetic inputs: random prompt ids for both branches, N(0,1) latent
    g = torch.Generator(device=dev).manual_seed(1234)
    ids_c = torch.randint(0, cfg.vocab_size, (1, args.text_len), generator=g, device=dev)
    ids_u = torch.randint(0, cfg.vocab_size, (1, args.text_len), generator=g, device=dev)
    total_steps = args.warmup + args.steps + 1 + args.e2e_steps + 1
    sc = SamplingConfig(num_steps=max(35, total_steps), guidance=args.guidance, shift=10.0, scheduler="euler", seed=0)
    st = pipe.engine.make_state(ids_c, ids_u, grid)
    x = pipe.begin(st, sc)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step_i = 0
    for _ in range(args.warmup):
        x = pipe.step(x, step_i); step_i += 1
    sync()
    ops.check_status()
    launches0 = ops.launch_count()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    torch.cuda.cudart().cudaProfilerStart()  # lets a profiler started with --profile-from-start off see only the timed steps
    e0.record()
    for _ in range(args.steps):
        x = pipe.step(x, step_i); step_i += 1
    e1.record()
    sync()
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
    sync()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.e2e_steps):
        pipe.step_from_host(host_in, step_i, host_out); step_i += 1
        host_in, host_out = host_out, host_in
    e3.record()
    sync()
    e2e_ms = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3) / max(1, args.e2e_steps)
    ops.check_status()
    finite = bool(torch.isfinite(host_in).all())

    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        pub = PUBLISHED_S_PER_VIDEO.get(world) if args.model == "Cosmos3-Nano" else None   # the table is Nano's
        base_ms = None if pub is None else pub * 1e3 / PUBLISHED_STEPS
        rec = {
            "metric": f"dit_step_ms ({args.model} T2V {args.resolution}p, one guided denoise step: cond+uncond forward, CFG, Euler)",
            "value": round(ms, 3), "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 3), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None if base_ms is None else round(ms / base_ms, 4),
            "dtype": "bf16", "data": "synthetic (random token ids, N(0,1) latent, random-init weights)",
            "s_per_video_35_steps": round(ms * 35 / 1e3, 2),
            "config": {"model": cfg.name + (" (layer override: INVALID as headline)" if args.layers else ""),
                       "global_batch": 1, "seq_len": n_tokens + args.text_len, "video_tokens": n_tokens,
                       "text_tokens": args.text_len, "frames": args.frames, "resolution": f"{width}x{height}",
                       "layers": cfg.n_layers, "cfg_scale": args.guidance, "parallelism": mesh.describe(),
                       "l2": "inputs larger than L2 (16 GB weights + GBs of activations per step)",
                       "baseline_note": "published number is for the reference's own 189-frame model, whose "
                                        "compute per token is far below these dense stand-in shapes"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_ms, 3), "unit": "ms",
                    "h2d_bytes_per_step": int(host_in.numel() * 4), "d2h_bytes_per_step": int(host_out.numel() * 4)},
            "gpu_launches": int(launches),
            "finite_output": finite,
        }
        print(json.dumps(rec), flush=True)
    if world > 1:
        from cosmos_b200.parallel.runtime import finish
        finish(hard=(__name__ == "__main__"))
    return 0


if __name__ == "__main__":
    sys.exit(main())

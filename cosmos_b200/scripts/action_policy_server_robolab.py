"""Policy server: serves action chunks to a simulator or robot client over HTTP.

    python -m cosmos_b200.scripts.action_policy_server_robolab --port 8000 [--checkpoint-path Cosmos3-Nano]

(reference: cookbooks/cosmos3/generator/action/run_policy_with_cosmos_framework.md:59-99; the
reference's RoboLab client `policies/cosmos3/run.py --task ...` connects to this port.)
The model stays resident; every `POST /act` takes the current camera image(s), the task
instruction and optionally the proprioceptive state, denoises future video AND action tokens
jointly (policy mode) and returns the next action chunk.

    POST /act   {"instruction": str, "image": base64 PNG/JPEG or [H, W, 3] list, "state": [..] (optional),
                 "domain_name": "droid_lerobot", "action_chunk_size": 16, "num_steps": 10, "seed": 0}
             -> {"action": [[...], ...], "shape": [chunk, D], "latency_ms": float}
    POST /reset -> {"ok": true}      GET /health -> {"status": "ok"}
"""
from __future__ import annotations

import argparse
import base64
import io
import time

import numpy as np
import torch

from ..config import SamplingConfig
from ..data.vfm.action.av_dataset import DOMAIN_ACTION_DIM, DOMAIN_DEFAULTS


class PolicyRunner:
    def __init__(self, pipe):
        self.pipe = pipe
        self.calls = 0

    def reset(self) -> None:
        self.calls = 0

    @staticmethod
    def decode_image(img) -> np.ndarray:
        if isinstance(img, str):
            from PIL import Image
            return np.asarray(Image.open(io.BytesIO(base64.b64decode(img.split(",")[-1]))).convert("RGB"))
        return np.asarray(img, dtype=np.uint8)

    def act(self, req: dict) -> dict:
        t0 = time.time()
        dom = req.get("domain_name", "droid_lerobot")
        defaults = DOMAIN_DEFAULTS.get(dom, {})
        chunk = int(req.get("action_chunk_size", defaults.get("action_chunk_size", 16)))
        size = int(req.get("image_size", defaults.get("image_size", 256)))
        adim = int(req.get("raw_action_dim", DOMAIN_ACTION_DIM.get(dom, 10)))
        image = self.decode_image(req["image"])
        from ..config import resolve_size
        w, h = resolve_size(str(size)) if str(size) in ("256", "480", "720") else (size, size)
        steps = int(req.get("num_steps", 10))
        sc = SamplingConfig(num_steps=steps, guidance=float(req.get("guidance", 1.0)), shift=10.0,
                            seed=int(req.get("seed", self.calls)), scheduler="euler")
        out = self.pipe(prompt=req.get("instruction", ""), image=image, num_frames=chunk + 1, height=h, width=w,
                        fps=int(defaults.get("fps", 15)), num_inference_steps=steps, guidance_scale=sc.guidance,
                        sampling=sc, domain=list(self.pipe.cfg.action_domains).index(dom), action_dim=adim,
                        n_action=chunk, denoise_action=True)
        self.calls += 1
        act = np.asarray(out.action, dtype=np.float32)
        return {"action": act.tolist(), "shape": list(act.shape), "latency_ms": (time.time() - t0) * 1e3}


def create_app(runner: PolicyRunner):
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="cosmos_b200 policy server")

    @app.get("/health")
    def health():
        return {"status": "ok"}

    @app.post("/reset")
    def reset():
        runner.reset()
        return {"ok": True}

    @app.post("/act")
    def act(req: dict):
        try:
            return runner.act(req)
        except KeyError as e:
            raise HTTPException(400, f"missing field {e}")

    return app


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--checkpoint-path", default="Cosmos3-Nano")
    ap.add_argument("--no-guardrails", action="store_true")
    args = ap.parse_args(argv)
    import uvicorn

    from ..pipeline import Cosmos3OmniPipeline

    dev = "cuda" if torch.cuda.is_available() else None
    pipe = Cosmos3OmniPipeline.from_pretrained(args.checkpoint_path, torch_dtype=torch.bfloat16 if dev else torch.float32,
                                               device_map=dev, enable_safety_checker=not args.no_guardrails)
    uvicorn.run(create_app(PolicyRunner(pipe)), host=args.host, port=args.port)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

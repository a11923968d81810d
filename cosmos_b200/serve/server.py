"""OpenAI-compatible HTTP server with a resident model (FastAPI).

Endpoints and fields follow the reference's serving surfaces (reference README.md:293-392,453-575;
cookbooks/cosmos3/generator/audiovisual/run_with_vllm_omni.ipynb:408-449;
action/run_fd_with_vllm.ipynb:361-440; action/README.md:100-104):

  POST /v1/images/generations   JSON  {prompt,size,n,num_inference_steps,guidance_scale,flow_shift,seed,extra_args}
                                 -> {"data":[{"b64_json": PNG}]}
  POST /v1/videos/sync          multipart form -> MP4 bytes
  POST /v1/videos               multipart form -> {"id"} (async job; actions via extra_params)
  GET  /v1/videos/{id}          -> {"status","progress","action":{data,shape,dtype}}
  GET  /v1/videos/{id}/content  -> MP4 bytes
  POST /v1/chat/completions     OpenAI chat (image_url / video_url / text parts; top_k, repetition_penalty)
  GET  /v1/models, /health, /v1/health/ready

The model stays resident; autoregressive action chunks loop in-process instead of reloading the
model per chunk. Generation jobs run on one worker thread (max_num_seqs 1 for the Generator, as in
the reference's deploy config, README.md:405-417); serving metrics (TTFT, request latency, output
tokens/s) are exported at /metrics.
"""
from __future__ import annotations

import base64
import io
import json
import os
import tempfile
import threading
import time
import uuid
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from ..config import DecodingConfig, SamplingConfig
from ..io import media, mp4
from ..utils.tokenizer import video_layout

try:  # module-level so that FastAPI can resolve the (string) annotations of the route handlers
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, Response
except ImportError:  # the endpoint logic in Cosmos3Server stays usable without FastAPI
    FastAPI = HTTPException = Request = JSONResponse = Response = None


@dataclass
class Job:
    id: str
    status: str = "queued"       # queued | in_progress | completed | failed | cancelled
    progress: int = 0
    error: Optional[str] = None
    video_path: Optional[str] = None
    action: Optional[np.ndarray] = None
    created: float = field(default_factory=time.time)


class Metrics:
    def __init__(self):
        self.lock = threading.Lock()
        self.requests = 0
        self.ttft_ms: List[float] = []
        self.latency_ms: List[float] = []
        self.output_tokens = 0
        self.t_first = None

    def record(self, ttft_ms: Optional[float], latency_ms: float, out_tokens: int = 0):
        with self.lock:
            self.requests += 1
            self.t_first = self.t_first or time.time()
            if ttft_ms is not None:
                self.ttft_ms.append(ttft_ms)
            self.latency_ms.append(latency_ms)
            self.output_tokens += out_tokens

    def snapshot(self) -> Dict[str, Any]:
        with self.lock:
            span = max(time.time() - (self.t_first or time.time()), 1e-9)
            avg = lambda v: (sum(v) / len(v)) if v else None  # noqa: E731
            return {"requests": self.requests, "avg_ttft_ms": avg(self.ttft_ms),
                    "avg_request_latency_ms": avg(self.latency_ms),
                    "output_token_throughput_per_s": self.output_tokens / span,
                    "request_throughput_per_s": self.requests / span}


def prometheus_text(snapshot: Dict[str, Any], prefix: str = "cosmos_b200") -> str:
    """The metrics snapshot in the Prometheus text exposition format (one gauge per figure)."""
    lines = []
    for key, value in snapshot.items():
        name = f"{prefix}_{key}"
        lines.append(f"# TYPE {name} gauge")
        lines.append(f"{name} {0.0 if value is None else float(value):.6g}")
    return "\n".join(lines) + "\n"


def parse_size(size: str):
    w, h = size.lower().split("x")
    return int(w), int(h)


class Cosmos3Server:
    """Holds the pipeline/reasoner and implements the endpoint logic independent of FastAPI."""

    def __init__(self, pipe, reasoner=None, vit=None, model_name: str = "nvidia/Cosmos3-Nano",
                 guardrails_default: bool = True, allowed_local_media_path: str = "", batch_engine=None):
        self.pipe, self.reasoner, self.vit = pipe, reasoner, vit
        # serve/engine.py::EngineWorker: chat requests share decode steps (continuous batching)
        self.batch_engine = batch_engine
        self.model_name = model_name
        self.guardrails_default = guardrails_default
        # empty = requests may not name files of this machine at all (media comes as data: URLs or uploads)
        self.allowed_root = Path(allowed_local_media_path).resolve() if allowed_local_media_path else None
        self.max_image_pixels = 12845056     # server-side ceiling per frame, whatever a request asks for (--max-image-pixels)
        self.max_video_frames = 32           # frames kept per clip unless the request names `max_frames`
        self.jobs: Dict[str, Job] = {}
        self.pool = ThreadPoolExecutor(max_workers=1)
        self.gen_lock = threading.Lock()
        self.metrics = Metrics()
        self.ready = True
        self.tmp = Path(tempfile.mkdtemp(prefix="cosmos_b200_jobs_"))

    # ------------------------------------------------------------------ generation
    def _generate(self, prompt: str, negative_prompt: Optional[str], width: int, height: int, num_frames: int,
                  fps: int, steps: int, guidance: float, flow_shift: float, seed: int, image=None, video=None,
                  generate_sound: bool = False, extra: Optional[dict] = None, job: Optional[Job] = None):
        extra = extra or {}
        if not getattr(self.pipe.transformer, "has_dm", hasattr(self.pipe.transformer, "dm")):
            raise ValueError("this server was started for the Reasoner only (no Generator tower is loaded)")
        sc = SamplingConfig(num_steps=steps, guidance=guidance, shift=flow_shift, seed=seed,
                            scheduler=extra.get("scheduler", "unipc"))
        kw: Dict[str, Any] = {}
        mode = extra.get("action_mode")
        if mode:
            from ..data.vfm.action.av_dataset import DOMAIN_ACTION_DIM
            dom = extra.get("domain_name", "av")
            kw["domain"] = list(self.pipe.cfg.action_domains).index(dom)
            kw["action_dim"] = int(extra.get("raw_action_dim") or DOMAIN_ACTION_DIM.get(dom, 9))
            chunk = int(extra.get("action_chunk_size", 16))
            num_frames = chunk + 1
            if mode == "forward_dynamics":
                act = extra.get("action")
                if act is None and extra.get("action_path"):
                    act = json.loads(self._local(extra["action_path"]).read_text())
                act = np.asarray(act, dtype=np.float32)
                if act.shape[0] > chunk and act.shape[0] % chunk == 0 and image is not None:
                    # several chunks of actions: rolled out in this process, each chunk from the last frame of the one before
                    kw["rollout"] = act
                kw["action"] = act[:chunk]
            else:  # inverse_dynamics / policy: actions are denoised
                kw["n_action"], kw["denoise_action"] = chunk, True
                if mode == "inverse_dynamics":
                    kw["condition_frame_indexes"] = list(range((num_frames - 1) // 4 + 1))
        if extra.get("condition_frame_indexes_vision"):
            kw["condition_frame_indexes"] = list(extra["condition_frame_indexes_vision"])
        for key in ("condition_video_keep", "max_sequence_length", "sound_duration"):
            if extra.get(key) not in (None, ""):
                kw[key] = extra[key]
        checker = self.pipe.safety_checker
        if not extra.get("guardrails", self.guardrails_default):
            self.pipe.safety_checker = None

        def cb(i, n):
            if job is not None:
                job.progress = int(100 * (i + 1) / n)

        try:
            with self.gen_lock:
                if "rollout" in kw:
                    acts = kw.pop("rollout")
                    n_chunks = acts.shape[0] // chunk
                    return self.pipe.forward_dynamics_rollout(
                        image, acts, chunk, kw["domain"], prompt, height, width, fps, seed,
                        callback=lambda k, n: cb(k, n_chunks), num_inference_steps=steps, guidance_scale=guidance,
                        sampling=sc, add_resolution_template=bool(extra.get("use_resolution_template", True)),
                        add_duration_template=bool(extra.get("use_duration_template", True)))
                return self.pipe(prompt=prompt, negative_prompt=negative_prompt, image=image, video=video,
                                 num_frames=num_frames, height=height, width=width, fps=fps,
                                 num_inference_steps=steps, guidance_scale=guidance, enable_sound=generate_sound,
                                 add_resolution_template=bool(extra.get("use_resolution_template", True)),
                                 add_duration_template=bool(extra.get("use_duration_template", True)),
                                 sampling=sc, callback=cb, output_type="np", **kw)
        finally:
            self.pipe.safety_checker = checker

    def _local(self, p: str) -> Path:
        if self.allowed_root is None:
            raise PermissionError("local media paths are disabled (start the server with --allowed-local-media-path DIR)")
        path = Path(p).resolve()
        if self.allowed_root not in path.parents and path != self.allowed_root:
            raise PermissionError(f"{p} is outside --allowed-local-media-path")
        return path

    def images_generations(self, body: dict) -> dict:
        t0 = time.time()
        w, h = parse_size(body.get("size", "1280x720"))
        out_data = []
        for k in range(int(body.get("n", 1))):
            out = self._generate(body["prompt"], body.get("negative_prompt"), w, h, 1, 24,
                                 int(body.get("num_inference_steps", 35)), float(body.get("guidance_scale", 6.0)),
                                 float(body.get("flow_shift", 10.0)), int(body.get("seed", 0)) + k,
                                 extra=body.get("extra_args"))
            buf = io.BytesIO()
            from PIL import Image
            Image.fromarray(out.video[0]).save(buf, format="PNG")
            out_data.append({"b64_json": base64.b64encode(buf.getvalue()).decode()})
        self.metrics.record(None, (time.time() - t0) * 1e3)
        return {"created": int(t0), "data": out_data}

    def _video_request(self, form: dict, ref_bytes: Optional[bytes], ref_name: str, job: Optional[Job]) -> Job:
        job = job or Job(id="sync")
        job.status = "in_progress"
        try:
            w, h = parse_size(form.get("size", "1280x720"))
            extra = form.get("extra_params") or {}
            if isinstance(extra, str):
                extra = json.loads(extra) if extra else {}
            image = video = None
            ref_tmp = None
            if ref_bytes:
                p = ref_tmp = self.tmp / f"{uuid.uuid4().hex}_{Path(ref_name or 'ref.bin').name}"
                p.write_bytes(ref_bytes)
                if p.suffix.lower() in (".png", ".jpg", ".jpeg", ".webp", ".bmp"):
                    image = str(p)
                else:
                    video = str(p)
            action_mode = bool(extra.get("action_mode"))
            for key, cast in (("max_sequence_length", int), ("sound_duration", float)):  # top-level form fields
                if form.get(key) not in (None, ""):
                    extra = {**extra, key: cast(form[key])}
            out = self._generate(form.get("prompt", ""), form.get("negative_prompt") or None, w, h,
                                 int(form.get("num_frames", 189)), int(form.get("fps", 24)),
                                 int(form.get("num_inference_steps", 30 if action_mode else 35)),
                                 float(form.get("guidance_scale", 1.0 if action_mode else 6.0)),
                                 float(form.get("flow_shift", 10.0)), int(form.get("seed", 0)), image, video,
                                 str(form.get("generate_sound", "false")).lower() == "true", extra, job)
            path = self.tmp / f"{job.id}_{uuid.uuid4().hex}.mp4"
            frames = out.video if out.video.ndim == 4 else out.video[None]
            media.write_video(path, frames, int(form.get("fps", 24)), 8, out.sound,
                              self.pipe.sound_tokenizer.config.sampling_rate)
            job.video_path, job.action = str(path), out.action
            job.status, job.progress = "completed", 100
        except Exception as e:  # noqa: BLE001 - reported through the job status
            job.status, job.error = "failed", f"{type(e).__name__}: {e}"
        finally:
            if ref_tmp is not None:
                ref_tmp.unlink(missing_ok=True)   # the uploaded reference is only needed while the job runs
        return job

    def videos_sync(self, form: dict, ref_bytes=None, ref_name="") -> bytes:
        t0 = time.time()
        job = self._video_request(form, ref_bytes, ref_name, None)
        if job.status != "completed":
            raise RuntimeError(job.error or "generation failed")
        self.metrics.record(None, (time.time() - t0) * 1e3)
        data = Path(job.video_path).read_bytes()
        Path(job.video_path).unlink(missing_ok=True)   # a synchronous result is returned once and not kept
        return data

    def videos_submit(self, form: dict, ref_bytes=None, ref_name="") -> dict:
        job = Job(id=f"video_{uuid.uuid4().hex[:16]}")
        self.jobs[job.id] = job
        self.pool.submit(self._video_request, form, ref_bytes, ref_name, job)
        return {"id": job.id, "object": "video", "status": job.status}

    def videos_status(self, job_id: str) -> dict:
        job = self.jobs[job_id]
        out = {"id": job.id, "object": "video", "status": job.status, "progress": job.progress}
        if job.error:
            out["error"] = {"message": job.error}
        if job.action is not None:
            a = np.asarray(job.action, dtype=np.float32)
            out["action"] = {"data": a.tolist(), "shape": list(a.shape), "dtype": "float32"}
        return out

    def videos_cancel(self, job_id: str) -> dict:
        job = self.jobs[job_id]
        if job.status == "queued":
            job.status = "cancelled"
        return self.videos_status(job_id)

    # ------------------------------------------------------------------ chat
    def chat_stream(self, body: dict):
        """Server-sent events for `"stream": true`: one `chat.completion.chunk` per piece of decoded text as
        the tokens come out of the decode batch, a last chunk with the finish reason, then `[DONE]`."""
        import queue

        q: "queue.Queue" = queue.Queue()
        cid, t0 = f"chatcmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        model = body.get("model", self.model_name)
        result: dict = {}

        def run():
            try:
                result["final"] = self.chat_completions(body, on_token=q.put)
            except Exception as e:  # noqa: BLE001 - reported to the client as an error event
                result["error"] = f"{type(e).__name__}: {e}"
            q.put(None)

        threading.Thread(target=run, daemon=True).start()

        def chunk(delta: dict, finish=None) -> str:
            return "data: " + json.dumps({"id": cid, "object": "chat.completion.chunk", "created": t0, "model": model,
                                          "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}) + "\n\n"

        tok = self.pipe.tokenizer
        ids: List[int] = []
        sent = ""
        stops, stopped = self._stops(body), False
        hold = max((len(s) for s in stops), default=1) - 1      # characters that could still become a stop string
        yield chunk({"role": "assistant", "content": ""})
        while True:
            t = q.get()
            if t is None:
                break
            if stopped:
                continue
            ids.append(int(t))
            text = tok.decode(ids)
            if text.endswith("\ufffd"):                          # hold back an incomplete multi-byte character
                continue
            text, stopped = self._cut_at_stop(text, stops)
            visible = text if stopped else text[:max(len(sent), len(text) - hold)]
            if len(visible) > len(sent):
                yield chunk({"content": visible[len(sent):]})
                sent = visible
        if not stopped and "final" in result:                      # what was held back in case it began a stop string
            rest = result["final"]["choices"][0]["message"]["content"]
            if len(rest) > len(sent) and rest.startswith(sent):
                yield chunk({"content": rest[len(sent):]})
        if "error" in result:
            yield "data: " + json.dumps({"error": {"message": result["error"]}}) + "\n\n"
        else:
            yield chunk({}, result["final"]["choices"][0]["finish_reason"])
        yield "data: [DONE]\n\n"

    @staticmethod
    def _stops(body: dict) -> List[str]:
        stop = body.get("stop")
        return [] if not stop else ([stop] if isinstance(stop, str) else [s for s in stop if s])

    @staticmethod
    def _cut_at_stop(text: str, stops: List[str]):
        """(text up to the first stop string, whether one was found)."""
        hits = [i for i in (text.find(s) for s in stops) if i >= 0]
        return (text[:min(hits)], True) if hits else (text, False)

    def chat_completions(self, body: dict, on_token=None) -> dict:
        """OpenAI chat completion. `stop` (a string or a list) ends the answer before the first stop string."""
        out = self._chat_completions(body, on_token)
        stops = self._stops(body)
        if stops:
            choice = out["choices"][0]
            choice["message"]["content"], found = self._cut_at_stop(choice["message"]["content"], stops)
            if found:
                choice["finish_reason"] = "stop"
        return out

    def _chat_completions(self, body: dict, on_token=None) -> dict:
        if self.reasoner is None:
            raise RuntimeError("this server was started without the Reasoner")
        t0 = time.time()
        tok = self.pipe.tokenizer
        messages = body["messages"]
        # The OpenAI client merges `extra_body` into the top level of the request; raw HTTP callers may nest it.
        extra = {k: body[k] for k in ("mm_processor_kwargs", "media_io_kwargs") if k in body}
        extra.update(body.get("extra_body") or {})
        vision_embeds, grids, n_vis, norm_msgs, deep = [], [], [], [], []
        has_video = False
        dev = self.pipe.device
        for m in messages:
            content = m["content"]
            if isinstance(content, list):
                parts = []
                for part in content:
                    kind = part.get("type")
                    if kind in ("image_url", "video_url"):
                        frames, times = self._load_media(part[kind]["url"], kind == "video_url", extra)
                        emb, grid, ds = self._encode_vision(frames, dev, (extra.get("mm_processor_kwargs") or {}).get("size"))
                        vision_embeds.append(emb)
                        deep.append(ds)
                        if kind == "video_url":
                            # one vision segment (and one rotary grid) per temporal group, each behind its time stamp
                            has_video = True
                            grids.extend([(1, grid[1], grid[2])] * grid[0])
                            n_vis.append(video_layout(grid, times, self.pipe.cfg.vit_temporal_patch))
                        else:
                            grids.append(grid)
                            n_vis.append(grid[0] * grid[1] * grid[2])
                    parts.append(part)
                norm_msgs.append({"role": m["role"], "content": parts})
            else:
                norm_msgs.append(m)
        ids = tok.apply_chat_template(norm_msgs, True, n_vis)
        dc = DecodingConfig(max_new_tokens=int(body.get("max_tokens", body.get("max_completion_tokens", 4096))),
                            do_sample=float(body.get("temperature", 0.7)) > 0,
                            temperature=float(body.get("temperature", 0.7)), top_p=float(body.get("top_p", 0.8)),
                            top_k=int(body.get("top_k", extra.get("top_k", 20))),
                            repetition_penalty=float(body.get("repetition_penalty", extra.get("repetition_penalty", 1.0))),
                            presence_penalty=float(body.get("presence_penalty", 1.5)), seed=body.get("seed"))
        first = {}
        user_cb = on_token

        def on_token(_t):
            first.setdefault("t", time.time())
            if user_cb is not None:
                user_cb(_t)

        ve = torch.cat(vision_embeds) if vision_embeds else None
        # DeepStack features of all media items, level by level
        ds = [torch.cat([d[k] for d in deep]) for k in range(len(deep[0]))] if deep and deep[0] else None
        # image and video pads share one mask here: every pad position takes the next vision row
        pad_id = tok.video_pad_id if has_video else tok.image_pad_id
        if ve is not None and len({tok.image_pad_id, tok.video_pad_id}) == 2:
            ids = [pad_id if t in (tok.image_pad_id, tok.video_pad_id) else t for t in ids]
        if self.batch_engine is not None and dc.seed is None:
            # joins the running decode batch instead of taking the generation lock (sampling runs on the
            # device; a request that pins a seed takes the single-request path). A prompt with media is
            # prefilled on its own (vision rows spliced in, 3-D rotary ids, DeepStack features) and then decodes
            # with everybody else.
            extra_kw = {}
            if ve is not None:
                ids_t = torch.tensor([ids], dtype=torch.long, device=dev)
                vmask = ids_t == pad_id
                x = self.reasoner.embed(ids_t.clamp(max=self.pipe.cfg.vocab_size - 1), ve, vmask)
                extra_kw = dict(embeds=x[0], positions=self.reasoner.positions(ids_t, vmask, grids),
                                vision_mask=vmask[0], deepstack=ds)
            stops = self._stops(body)
            if stops:
                # the engine retires the request as soon as a stop string is complete instead of decoding to the limit
                seen_ids: List[int] = []
                inner = user_cb

                def user_cb(t, _inner=inner):
                    if _inner is not None:
                        _inner(t)
                    seen_ids.append(int(t))
                    return not self._cut_at_stop(tok.decode(seen_ids), stops)[1]
            r = self.batch_engine.submit(ids, dc.max_new_tokens, (tok.eos_id, tok.eot_id),
                                         temperature=dc.temperature if dc.do_sample else 0.0, top_k=dc.top_k,
                                         top_p=dc.top_p, presence_penalty=dc.presence_penalty,
                                         repetition_penalty=dc.repetition_penalty, on_token=user_cb,
                                         **extra_kw).result()
            t1 = time.time()
            self.metrics.record((r.t_first - t0) * 1e3, (t1 - t0) * 1e3, len(r.out))
            return {"id": f"chatcmpl-{uuid.uuid4().hex[:24]}", "object": "chat.completion", "created": int(t0),
                    "model": body.get("model", self.model_name),
                    "choices": [{"index": 0, "message": {"role": "assistant", "content": tok.decode(r.out)},
                                 "finish_reason": r.finish_reason}],
                    "usage": {"prompt_tokens": len(ids), "completion_tokens": len(r.out),
                              "total_tokens": len(ids) + len(r.out)}}
        with self.gen_lock:
            out_ids, usage = self.reasoner.generate(ids, dc, (tok.eos_id, tok.eot_id), ve, pad_id if ve is not None else None,
                                                    grids, on_token, deepstack=ds)
        text = tok.decode(out_ids)
        t1 = time.time()
        self.metrics.record((first.get("t", t1) - t0) * 1e3, (t1 - t0) * 1e3, usage["completion_tokens"])
        return {"id": f"chatcmpl-{uuid.uuid4().hex[:24]}", "object": "chat.completion", "created": int(t0),
                "model": body.get("model", self.model_name),
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text},
                             "finish_reason": "stop" if out_ids and out_ids[-1] in (tok.eos_id, tok.eot_id) else "length"}],
                "usage": {**usage, "total_tokens": usage["prompt_tokens"] + usage["completion_tokens"]}}

    def _load_media(self, url: str, is_video: bool, extra: dict):
        """Frames (and their times) of one media item of a chat request. `data:` URLs are decoded into a temporary file
        that is removed again before returning; `file://` URLs and bare paths are served only below
        --allowed-local-media-path (off by default); remote URLs are refused (this server fetches nothing)."""
        tmp = None
        try:
            if url.startswith("data:"):
                raw = base64.b64decode(url.split(",", 1)[1])
                suffix = ".mp4" if is_video else ".png"
                p = tmp = self.tmp / f"{uuid.uuid4().hex}{suffix}"
                p.write_bytes(raw)
            elif url.startswith(("http://", "https://")):
                raise ValueError("remote media URLs are not fetched by this server: send the media as a data: URL")
            elif url.startswith("file://"):
                p = self._local(url[7:])
            else:
                p = self._local(url)
            return self._read_media(p, is_video, extra)
        finally:
            if tmp is not None:
                tmp.unlink(missing_ok=True)

    def _read_media(self, p, is_video: bool, extra: dict):
        if not is_video:
            frames, _ = media.read_video(p, max_frames=1)
            return frames, [0.0]
        vk = (extra.get("media_io_kwargs") or {}).get("video", {})
        mk = extra.get("mm_processor_kwargs") or {}
        limit = int(vk.get("max_frames", mk.get("max_frames", self.max_video_frames)))
        if int(vk.get("num_frames", 0)) > 0:
            frames, times, _ = media.sample_video(p, num_frames=int(vk["num_frames"]), limit=limit)
        elif vk.get("num_frames") == -1 or mk.get("do_sample_frames") is False:
            frames, times, _ = media.sample_video(p, limit=limit)   # the client pre-sampled the clip: keep every frame
        else:
            frames, times, _ = media.sample_video(p, fps=float(vk.get("fps", mk.get("fps", 2))), limit=limit)
        return frames, times                                  # frames and their times in the source clip

    def _encode_vision(self, frames: np.ndarray, dev, size: Optional[dict] = None):
        from PIL import Image
        from ..models.vae import CausalVideoVAE
        unit = self.pipe.cfg.vit_patch * self.pipe.cfg.vit_spatial_merge
        size = size or {}
        # pixel bounds per frame: the request's, else 3136 .. 12845056 for an image (reference README.md:574) and, for
        # a clip, an equal share of 25165824 pixels over its frames (the Qwen3-VL video default)
        most = 12845056 if frames.shape[0] == 1 else min(12845056, 25165824 // frames.shape[0])
        most = min(int(size.get("longest_edge", most)), self.max_image_pixels)
        h, w = smart_resize(frames.shape[1], frames.shape[2], unit, min(int(size.get("shortest_edge", 3136)), most), most)
        fr = np.stack([np.asarray(Image.fromarray(f).resize((w, h))) for f in frames])
        vid = CausalVideoVAE.from_uint8(torch.from_numpy(fr)[None])[0].permute(1, 0, 2, 3).to(dev)
        with torch.no_grad():
            return self.vit(vid, return_deepstack=True)

    def models(self) -> dict:
        return {"object": "list", "data": [{"id": self.model_name, "object": "model", "owned_by": "cosmos_b200"}]}


def smart_resize(h: int, w: int, unit: int, min_pixels: int, max_pixels: int, max_side: Optional[int] = None):
    """Target (height, width) for the vision encoder: multiples of `unit` (patch x spatial merge), aspect
    ratio kept, pixel count within [min_pixels, max_pixels] (the `size.shortest_edge` / `size.longest_edge`
    bounds of `mm_processor_kwargs`, reference README.md:574), each side at most `max_side`."""
    import math
    hb, wb = max(unit, round(h / unit) * unit), max(unit, round(w / unit) * unit)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb, wb = max(unit, math.floor(h / beta / unit) * unit), max(unit, math.floor(w / beta / unit) * unit)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb, wb = math.ceil(h * beta / unit) * unit, math.ceil(w * beta / unit) * unit
    if max_side:
        hb, wb = min(hb, max_side), min(wb, max_side)
    return hb, wb


def create_app(server: Cosmos3Server):
    if FastAPI is None:
        raise RuntimeError("fastapi is not installed")
    app = FastAPI(title="cosmos_b200")

    async def _form(request: Request):
        ctype = request.headers.get("content-type", "")
        if ctype.startswith("application/json"):
            return await request.json(), None, ""
        form = await request.form()
        fields, ref, name = {}, None, ""
        for k, v in form.multi_items():
            if hasattr(v, "read"):
                ref, name = await v.read(), getattr(v, "filename", "") or ""
            else:
                fields[k] = v
        return fields, ref, name

    @app.get("/health")
    @app.get("/v1/health/ready")
    def health():
        if not server.ready:
            raise HTTPException(503, "loading")
        return {"status": "ok"}

    @app.get("/v1/models")
    def models():
        return server.models()

    @app.get("/metrics")
    def metrics(request: Request):
        """JSON by default; `?format=prometheus` (or a scraper's `Accept: text/plain`) gives the text exposition format."""
        snap = server.metrics.snapshot()
        if request.query_params.get("format") == "prometheus" or "text/plain" in request.headers.get("accept", ""):
            return Response(prometheus_text(snap), media_type="text/plain; version=0.0.4")
        return snap

    @app.post("/v1/images/generations")
    async def images(request: Request):
        try:
            return server.images_generations(await request.json())
        except Exception as e:  # noqa: BLE001
            raise HTTPException(400, f"{type(e).__name__}: {e}")

    @app.post("/v1/videos/sync")
    async def videos_sync(request: Request):
        fields, ref, name = await _form(request)
        try:
            return Response(server.videos_sync(fields, ref, name), media_type="video/mp4")
        except Exception as e:  # noqa: BLE001
            raise HTTPException(400, f"{type(e).__name__}: {e}")

    @app.post("/v1/videos")
    async def videos(request: Request):
        fields, ref, name = await _form(request)
        return server.videos_submit(fields, ref, name)

    @app.get("/v1/videos/{job_id}")
    def video_status(job_id: str):
        if job_id not in server.jobs:
            raise HTTPException(404, "no such job")
        return server.videos_status(job_id)

    @app.delete("/v1/videos/{job_id}")
    def video_cancel(job_id: str):
        if job_id not in server.jobs:
            raise HTTPException(404, "no such job")
        return server.videos_cancel(job_id)

    @app.get("/v1/videos/{job_id}/content")
    def video_content(job_id: str):
        job = server.jobs.get(job_id)
        if job is None:
            raise HTTPException(404, "no such job")
        if job.status != "completed":
            raise HTTPException(409, f"job is {job.status}")
        return Response(Path(job.video_path).read_bytes(), media_type="video/mp4")

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        try:
            body = await request.json()
            if body.get("stream"):
                from starlette.responses import StreamingResponse
                return StreamingResponse(server.chat_stream(body), media_type="text/event-stream")
            return server.chat_completions(body)
        except Exception as e:  # noqa: BLE001
            raise HTTPException(400, f"{type(e).__name__}: {e}")

    return app


def apply_deploy_config(args) -> None:
    """Folds a deploy-config YAML into the parsed arguments: `stages[*].model_config.guardrails: false`
    switches the guardrails off, `model_class_name` overrides the flag of the same name."""
    if not getattr(args, "deploy_config", None):
        return
    import yaml

    with open(args.deploy_config) as f:
        cfg = yaml.safe_load(f) or {}
    for stage in cfg.get("stages") or []:
        mc = stage.get("model_config") or {}
        if mc.get("guardrails") is False:
            args.no_guardrails = True
        if stage.get("model_class_name"):
            args.model_class_name = stage["model_class_name"]


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="cosmos_b200 serve (Generator + Reasoner)")
    ap.add_argument("model", nargs="?", default="nvidia/Cosmos3-Nano")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--omni", action="store_true", help="accepted for CLI compatibility")
    ap.add_argument("--model-class-name", default="Cosmos3OmniDiffusersPipeline")
    ap.add_argument("--allowed-local-media-path", default="",
                    help="directory below which chat requests may name local files (file:// URLs or paths); "
                         "empty (default) = no local file access")
    ap.add_argument("--init-timeout", type=int, default=1800)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--cfg-parallel-size", type=int, default=1)
    ap.add_argument("--ulysses-degree", type=int, default=1)
    ap.add_argument("--enable-layerwise-offload", action="store_true")
    ap.add_argument("--no-guardrails", "--cosmos3-no-guardrails", dest="no_guardrails", action="store_true",
                    help="never load the guardrail models (per-request overrides cannot turn them back on)")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--deploy-config", default=None,
                    help="YAML with stages[].model_config.{guardrails, offload_guardrail_models} "
                         "(reference README.md:405-423)")
    ap.add_argument("--mm-encoder-tp-mode", default="data", choices=["data", "weights"],
                    help="the vision encoder is replicated on every rank (data); accepted for CLI compatibility")
    ap.add_argument("--media-io-kwargs", default=None, help='JSON, e.g. {"video": {"num_frames": -1}}')
    ap.add_argument("--max-num-seqs", type=int, default=8,
                    help="decode slots of the continuous-batching engine for chat requests (0 = off)")
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--hf-overrides", default=None,
                    help='JSON; {"architectures": ["Cosmos3ReasonerForConditionalGeneration"]} serves the Reasoner only '
                         "(the Generator tower is not built)")
    ap.add_argument("--async-scheduling", action="store_true",
                    help="accepted for CLI compatibility: the batching engine always steps in its own thread")
    ap.add_argument("--max-image-pixels", type=int, default=12845056,
                    help="ceiling on the pixels per image / video frame after resizing, whatever a request asks for")
    args = ap.parse_args(argv)
    apply_deploy_config(args)
    import uvicorn

    from ..models.reasoner import ReasonerEngine
    from ..pipeline import Cosmos3OmniPipeline

    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}" if torch.cuda.is_available() else None
    dtype = torch.bfloat16 if (dev and args.dtype == "bf16") else torch.float32
    over = json.loads(args.hf_overrides) if args.hf_overrides else {}
    reasoner_only = "Cosmos3ReasonerForConditionalGeneration" in (over.get("architectures") or [])
    pipe = Cosmos3OmniPipeline.from_pretrained(args.model, torch_dtype=dtype, device_map=dev,
                                               enable_safety_checker=not args.no_guardrails,
                                               towers=("ar",) if reasoner_only else ("ar", "dm"))
    vit = pipe.vision_encoder()
    worker = None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    group = None
    if world > 1:
        # launched with torchrun: the Reasoner's decode batch is tensor-parallel over all ranks; rank 0 serves HTTP
        # (and runs the Generator endpoints on its own GPU), the other ranks mirror its engine steps
        import torch.distributed as dist

        from ..parallel.runtime import init_distributed
        from ..config import ParallelConfig
        init_distributed(world, int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
                         pc=ParallelConfig(tp=world))
        group = dist.group.WORLD
        if args.max_num_seqs <= 0:
            raise SystemExit("a multi-rank server needs --max-num-seqs > 0 (the tensor-parallel engine)")
    if args.max_num_seqs > 0:
        from .engine import BatchEngine, EngineWorker
        engine = BatchEngine(pipe.transformer, max_batch=args.max_num_seqs, max_len=args.max_model_len, group=group)
        if world > 1 and int(os.environ.get("RANK", "0")) != 0:
            engine.follow()
            return 0
        worker = EngineWorker(engine)
    server = Cosmos3Server(pipe, ReasonerEngine(pipe.transformer, vit), vit, args.model, not args.no_guardrails,
                           args.allowed_local_media_path, batch_engine=worker)
    server.max_image_pixels = args.max_image_pixels
    uvicorn.run(create_app(server), host=args.host, port=args.port, log_level="info")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

"""HTTP surface on CPU with the tiny model: every endpoint of the serving table once."""
import base64
import io
import json
import time

import numpy as np
import pytest
import torch

fastapi = pytest.importorskip("fastapi")
pytest.importorskip("httpx")
from fastapi.testclient import TestClient  # noqa: E402

from cosmos_b200.io import mp4  # noqa: E402
from cosmos_b200.models.reasoner import ReasonerEngine  # noqa: E402
from cosmos_b200.models.vit import VisionEncoder  # noqa: E402
from cosmos_b200.pipeline import Cosmos3OmniPipeline  # noqa: E402
from cosmos_b200.serve.server import Cosmos3Server, create_app  # noqa: E402


@pytest.fixture(scope="module")
def client():
    torch.manual_seed(0)
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=32, n_layers=2))
    vit = VisionEncoder(pipe.cfg).eval()
    srv = Cosmos3Server(pipe, ReasonerEngine(pipe.transformer, vit), vit, "nvidia/Cosmos3-Nano",
                        allowed_local_media_path="/")
    return TestClient(create_app(srv))


def test_local_and_remote_media_are_refused_by_default_and_temp_files_do_not_pile_up(tmp_path):
    """Without --allowed-local-media-path a request cannot make the server open files of its machine; remote URLs are
    never fetched; media sent as data: URLs leaves nothing behind in the server's scratch directory."""
    import base64
    import io
    import os

    from PIL import Image
    torch.manual_seed(0)
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=32, n_layers=1))
    vit = VisionEncoder(pipe.cfg).eval()
    srv = Cosmos3Server(pipe, ReasonerEngine(pipe.transformer, vit), vit, "nvidia/Cosmos3-Nano")
    c = TestClient(create_app(srv), raise_server_exceptions=False)
    img = tmp_path / "a.png"
    Image.new("RGB", (32, 32), (200, 10, 10)).save(img)

    def ask(url):
        body = {"max_tokens": 2, "temperature": 0.0,
                "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}},
                                                          {"type": "text", "text": "what is this?"}]}]}
        return c.post("/v1/chat/completions", json=body)

    for url in (f"file://{img}", str(img), "https://example.com/a.png"):
        assert ask(url).status_code >= 400, url
    buf = io.BytesIO()
    Image.open(img).save(buf, format="PNG")
    ok = ask("data:image/png;base64," + base64.b64encode(buf.getvalue()).decode())
    assert ok.status_code == 200, ok.text
    assert os.listdir(srv.tmp) == []
    # opting in to a directory serves files below it and nothing else
    srv2 = Cosmos3Server(pipe, ReasonerEngine(pipe.transformer, vit), vit, "nvidia/Cosmos3-Nano",
                         allowed_local_media_path=str(tmp_path))
    assert srv2._local(str(img)) == img.resolve()
    with pytest.raises(PermissionError):
        srv2._local("/etc/hostname")


def test_health_and_models(client):
    assert client.get("/health").status_code == 200
    assert client.get("/v1/health/ready").json()["status"] == "ok"
    assert client.get("/v1/models").json()["data"][0]["id"] == "nvidia/Cosmos3-Nano"


def test_images_generations(client):
    r = client.post("/v1/images/generations", json={"prompt": "a cat", "size": "64x64", "n": 1,
                                                    "num_inference_steps": 2, "guidance_scale": 4.0, "flow_shift": 3.0,
                                                    "seed": 1, "extra_args": {"use_resolution_template": False}})
    assert r.status_code == 200, r.text
    png = base64.b64decode(r.json()["data"][0]["b64_json"])
    assert png[:8] == b"\x89PNG\r\n\x1a\n"


def test_videos_sync_returns_mp4(client):
    r = client.post("/v1/videos/sync", data={"prompt": "a robot", "negative_prompt": "blurry", "size": "64x64",
                                             "num_frames": "5", "fps": "24", "num_inference_steps": "2",
                                             "guidance_scale": "3.0", "flow_shift": "3.0", "seed": "0"})
    assert r.status_code == 200, r.text
    assert r.content[4:8] == b"ftyp"


def test_async_action_job_forward_and_inverse(client, tmp_path):
    img = io.BytesIO()
    from PIL import Image
    Image.fromarray((np.random.rand(64, 64, 3) * 255).astype(np.uint8)).save(img, format="PNG")
    extra = {"action_mode": "forward_dynamics", "domain_name": "av", "raw_action_dim": 9, "action_chunk_size": 4,
             "action": np.zeros((4, 9)).tolist(), "guardrails": False}
    r = client.post("/v1/videos", data={"prompt": "drive", "size": "64x64", "num_inference_steps": "2",
                                        "extra_params": json.dumps(extra)},
                    files={"input_reference": ("frame.png", img.getvalue(), "image/png")})
    jid = r.json()["id"]
    for _ in range(200):
        st = client.get(f"/v1/videos/{jid}").json()
        if st["status"] in ("completed", "failed"):
            break
        time.sleep(0.1)
    assert st["status"] == "completed", st
    content = client.get(f"/v1/videos/{jid}/content")
    assert content.status_code == 200 and content.content[4:8] == b"ftyp"
    clip = tmp_path / "clip.mp4"
    clip.write_bytes(content.content)
    frames, _ = mp4.read_mp4_mjpeg(clip)
    assert frames.shape[0] == 5
    extra = {"action_mode": "inverse_dynamics", "domain_name": "av", "raw_action_dim": 9, "action_chunk_size": 4}
    r = client.post("/v1/videos", data={"prompt": "drive", "size": "64x64", "num_inference_steps": "2",
                                        "extra_params": json.dumps(extra)},
                    files={"input_reference": ("clip.mp4", content.content, "video/mp4")})
    jid = r.json()["id"]
    for _ in range(200):
        st = client.get(f"/v1/videos/{jid}").json()
        if st["status"] in ("completed", "failed"):
            break
        time.sleep(0.1)
    assert st["status"] == "completed", st
    assert st["action"]["shape"] == [4, 9] and st["action"]["dtype"] == "float32"
    assert client.get("/v1/videos/nope").status_code == 404


def test_chat_completions_text_and_image(client):
    img = io.BytesIO()
    from PIL import Image
    Image.fromarray((np.random.rand(64, 64, 3) * 255).astype(np.uint8)).save(img, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(img.getvalue()).decode()
    body = {"model": "nvidia/Cosmos3-Nano", "max_tokens": 5, "temperature": 0.0, "top_k": 20,
            "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}},
                                                       {"type": "text", "text": "What is in the image?"}]}]}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    out = r.json()
    assert out["choices"][0]["message"]["role"] == "assistant"
    assert out["usage"]["completion_tokens"] <= 5 and out["usage"]["prompt_tokens"] > 4
    m = client.get("/metrics").json()
    assert m["requests"] >= 1 and m["avg_request_latency_ms"] > 0


def test_deploy_config_switches_guardrails_off(tmp_path):
    import argparse
    from cosmos_b200.serve.server import apply_deploy_config

    cfg = tmp_path / "no_guardrails.yaml"
    cfg.write_text("async_chunk: false\nstages:\n  - stage_id: 0\n    max_num_seqs: 1\n"
                   "    model_class_name: Cosmos3OmniDiffusersPipeline\n    model_config:\n      guardrails: false\n"
                   "      offload_guardrail_models: false\n")
    args = argparse.Namespace(deploy_config=str(cfg), no_guardrails=False, model_class_name="x")
    apply_deploy_config(args)
    assert args.no_guardrails is True and args.model_class_name == "Cosmos3OmniDiffusersPipeline"
    args = argparse.Namespace(deploy_config=None, no_guardrails=False, model_class_name="x")
    apply_deploy_config(args)
    assert args.no_guardrails is False


def test_concurrent_text_chats_share_the_batching_engine():
    """Text-only greedy chat requests go through the continuous-batching engine: eight concurrent HTTP
    requests complete in fewer decode steps than their token budgets add up to."""
    from concurrent.futures import ThreadPoolExecutor

    from cosmos_b200.serve.engine import BatchEngine, EngineWorker

    torch.manual_seed(0)
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(max_text_len=32, n_layers=2))
    worker = EngineWorker(BatchEngine(pipe.transformer, max_batch=4, max_len=256, page_size=4, use_graph=False))
    try:
        srv = Cosmos3Server(pipe, ReasonerEngine(pipe.transformer, None), None, "nvidia/Cosmos3-Nano",
                            batch_engine=worker)
        c = TestClient(create_app(srv))

        def ask(i):
            body = {"model": "nvidia/Cosmos3-Nano", "max_tokens": 6, "temperature": 0.0,
                    "messages": [{"role": "user", "content": f"question number {i}"}]}
            return c.post("/v1/chat/completions", json=body)

        with ThreadPoolExecutor(8) as ex:
            rs = list(ex.map(ask, range(8)))
        assert all(r.status_code == 200 for r in rs), [r.text for r in rs if r.status_code != 200]
        outs = [r.json() for r in rs]
        assert all(o["usage"]["completion_tokens"] <= 6 and o["choices"][0]["finish_reason"] in ("stop", "length")
                   for o in outs)
        total = sum(o["usage"]["completion_tokens"] for o in outs)
        assert worker.engine.steps < total
        # a request with an image goes through the same engine (prefilled alone, decoded with the batch)
        from cosmos_b200.models.vit import VisionEncoder
        from PIL import Image
        vit = VisionEncoder(pipe.cfg).eval()
        srv.vit, srv.reasoner = vit, ReasonerEngine(pipe.transformer, vit)
        img = io.BytesIO()
        Image.fromarray((np.random.rand(64, 64, 3) * 255).astype(np.uint8)).save(img, format="PNG")
        url = "data:image/png;base64," + base64.b64encode(img.getvalue()).decode()
        steps0 = worker.engine.steps
        r = c.post("/v1/chat/completions", json={"model": "nvidia/Cosmos3-Nano", "max_tokens": 4, "temperature": 0.7,
                   "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}},
                                                              {"type": "text", "text": "what is this?"}]}]})
        assert r.status_code == 200, r.text
        assert r.json()["usage"]["completion_tokens"] <= 4 and worker.engine.steps > steps0
    finally:
        worker.close()


def test_chat_streaming_sends_chunks_then_done(client):
    """`"stream": true`: server-sent events whose deltas add up to the non-streamed answer (greedy)."""
    body = {"model": "nvidia/Cosmos3-Nano", "max_tokens": 6, "temperature": 0.0,
            "messages": [{"role": "user", "content": "say something"}]}
    whole = client.post("/v1/chat/completions", json=body).json()
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as r:
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        events = [line[6:] for line in r.iter_lines() if line.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert all(c["object"] == "chat.completion.chunk" for c in chunks)
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    assert text == whole["choices"][0]["message"]["content"]
    assert chunks[-1]["choices"][0]["finish_reason"] in ("stop", "length")


def test_video_request_fields_sound_duration_sequence_length_and_keep(client, tmp_path):
    """`max_sequence_length`, `sound_duration`, `generate_sound` as form fields and `condition_video_keep`,
    `use_duration_template` inside `extra_params` (reference README.md:389-391)."""
    from cosmos_b200.io import media
    src = tmp_path / "src.mp4"
    media.write_video(src, (np.random.rand(9, 64, 64, 3) * 255).astype(np.uint8), 8, 8, None, 48000)
    extra = {"condition_frame_indexes_vision": [0, 1], "condition_video_keep": "last", "use_duration_template": False}
    with pytest.warns(UserWarning, match="truncated to max_sequence_length=8"):
        r = client.post("/v1/videos/sync",
                        data={"prompt": "a robot arm stacks red blocks on a table " * 4, "size": "64x64", "num_frames": "9",
                              "fps": "8", "num_inference_steps": "2", "guidance_scale": "1.0", "seed": "0",
                              "max_sequence_length": "8", "generate_sound": "true", "sound_duration": "0.5",
                              "extra_params": json.dumps(extra)},
                        files={"input_reference": ("src.mp4", src.read_bytes(), "video/mp4")})
    assert r.status_code == 200, r.text
    assert r.content[4:8] == b"ftyp"
    bad = client.post("/v1/videos/sync", data={"prompt": "x", "size": "64x64", "num_frames": "5", "num_inference_steps": "1",
                                               "extra_params": json.dumps({"condition_video_keep": "middle"})},
                      files={"input_reference": ("src.mp4", src.read_bytes(), "video/mp4")})
    assert bad.status_code >= 400


def test_chat_video_with_processor_kwargs(client, tmp_path):
    """`mm_processor_kwargs` {fps, do_sample_frames, size} and `media_io_kwargs` of a chat request."""
    from cosmos_b200.io import media
    from cosmos_b200.serve.server import smart_resize
    src = tmp_path / "clip.mp4"
    media.write_video(src, (np.random.rand(8, 96, 128, 3) * 255).astype(np.uint8), 8, 8, None, 48000)
    url = "data:video/mp4;base64," + base64.b64encode(src.read_bytes()).decode()
    usage = {}
    for mk in ({"fps": 4, "do_sample_frames": True}, {"do_sample_frames": False},
               {"fps": 4, "do_sample_frames": True, "size": {"shortest_edge": 1024, "longest_edge": 4096}}):
        body = {"max_tokens": 2, "temperature": 0.0, "mm_processor_kwargs": mk,
                "messages": [{"role": "user", "content": [{"type": "video_url", "video_url": {"url": url}},
                                                           {"type": "text", "text": "Describe the clip."}]}]}
        r = client.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        usage[json.dumps(mk)] = r.json()["usage"]["prompt_tokens"]
    n_sampled, n_all, n_small = usage.values()
    assert n_all > n_sampled > n_small  # every frame > 4 fps sampling > 4 fps with a tighter pixel bound
    assert smart_resize(96, 128, 32, 1024, 4096) == (32, 64)
    assert smart_resize(720, 1280, 32, 3136, 262144) == (384, 672)
    assert smart_resize(20, 20, 32, 3136, 10 ** 7) == (64, 64)


def test_chat_reads_a_real_h264_clip_from_the_reference_assets(client):
    """`video_url` pointing at one of the reference's own example clips (H.264), sampled at 4 frames per second as
    its notebooks do."""
    pytest.importorskip("cv2")
    from pathlib import Path
    clip = Path(__file__).resolve().parents[2] / "reference" / "cookbooks" / "cosmos3" / "reasoner" / "assets" / "video_caption.mp4"
    if not clip.exists():
        pytest.skip("reference assets not mounted")
    body = {"max_tokens": 3, "temperature": 0.0, "mm_processor_kwargs": {"fps": 4, "do_sample_frames": True},
            "messages": [{"role": "system", "content": "You are a helpful assistant."},
                         {"role": "user", "content": [{"type": "video_url", "video_url": {"url": f"file://{clip}"}},
                                                      {"type": "text", "text": "What's happening in this video?"}]}]}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    usage = r.json()["usage"]
    assert usage["prompt_tokens"] > 60 and 1 <= usage["completion_tokens"] <= 3      # vision rows of several frames


def test_chat_responses_parse_with_the_vllm_openai_schema(client):
    """The reference serves the Reasoner through vLLM's OpenAI-compatible server; this server's chat answers (plain
    and streamed) must parse with that server's own response models."""
    proto = pytest.importorskip("vllm.entrypoints.openai.chat_completion.protocol")
    body = {"model": "nvidia/Cosmos3-Nano", "max_tokens": 4, "temperature": 0.0,
            "messages": [{"role": "user", "content": "Describe a robot arm."}]}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    parsed = proto.ChatCompletionResponse.model_validate(r.json())
    assert parsed.choices[0].message.role == "assistant" and parsed.usage.completion_tokens <= 4
    assert parsed.object == "chat.completion" and parsed.choices[0].finish_reason in ("stop", "length")
    chunks = []
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as s:
        for line in s.iter_lines():
            if line.startswith("data: ") and line != "data: [DONE]":
                chunks.append(proto.ChatCompletionStreamResponse.model_validate(json.loads(line[6:])))
    assert chunks and chunks[0].object == "chat.completion.chunk"
    assert chunks[-1].choices[0].finish_reason in ("stop", "length")
    assert len({c.id for c in chunks}) == 1                              # one id for the whole stream


def test_reasoner_only_server_refuses_generator_requests():
    """`--hf-overrides '{"architectures": ["Cosmos3ReasonerForConditionalGeneration"]}'`: only the AR tower is
    built; chat works, Generator endpoints answer 400 with the reason."""
    torch.manual_seed(0)
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16), towers=("ar",),
                                               config_overrides=dict(max_text_len=32, n_layers=1))
    assert not pipe.transformer.has_dm
    vit = pipe.vision_encoder()
    c = TestClient(create_app(Cosmos3Server(pipe, ReasonerEngine(pipe.transformer, vit), vit, "nvidia/Cosmos3-Nano")))
    r = c.post("/v1/chat/completions", json={"max_tokens": 2, "temperature": 0.0, "messages": [{"role": "user", "content": "hi"}]})
    assert r.status_code == 200, r.text
    r = c.post("/v1/images/generations", json={"prompt": "a cat", "size": "64x64", "num_inference_steps": 1})
    assert r.status_code == 400 and "Reasoner only" in r.text
    r = c.post("/v1/videos/sync", data={"prompt": "x", "size": "64x64", "num_frames": "5", "num_inference_steps": "1"})
    assert r.status_code >= 400 and "Reasoner only" in r.text


def test_forward_dynamics_job_with_several_action_chunks_rolls_out_in_process(client, tmp_path):
    """12 actions with action_chunk_size 4 in one request: three chunks chained on the last frame, 13 frames back."""
    img = io.BytesIO()
    from PIL import Image
    Image.fromarray((np.random.rand(64, 64, 3) * 255).astype(np.uint8)).save(img, format="PNG")
    extra = {"action_mode": "forward_dynamics", "domain_name": "av", "raw_action_dim": 9, "action_chunk_size": 4,
             "action": (np.random.randn(12, 9) * 0.05).tolist(), "guardrails": False}
    r = client.post("/v1/videos", data={"prompt": "drive", "size": "64x64", "num_inference_steps": "1", "fps": "10",
                                        "extra_params": json.dumps(extra)},
                    files={"input_reference": ("frame.png", img.getvalue(), "image/png")})
    jid = r.json()["id"]
    for _ in range(300):
        st = client.get(f"/v1/videos/{jid}").json()
        if st["status"] in ("completed", "failed"):
            break
        time.sleep(0.1)
    assert st["status"] == "completed" and st["progress"] == 100, st
    clip = tmp_path / "rollout.mp4"
    clip.write_bytes(client.get(f"/v1/videos/{jid}/content").content)
    frames, fps = mp4.read_mp4_mjpeg(clip)
    assert frames.shape[0] == 13 and abs(fps - 10) < 1e-6


def test_stop_strings_end_the_answer_plain_and_streamed():
    """`stop`: the answer ends before the first stop string, also when the string arrives split over several streamed
    tokens; text that only looked like the beginning of a stop string is still delivered."""
    torch.manual_seed(0)
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16), towers=("ar",),
                                               config_overrides=dict(max_text_len=32, n_layers=1))
    srv = Cosmos3Server(pipe, ReasonerEngine(pipe.transformer, None), None, "nvidia/Cosmos3-Nano")
    answer = "The arm lifts the cube. END and more; almost EN done"

    def fake(body, on_token=None):                       # a model that says `answer`, one byte-token at a time
        for t in pipe.tokenizer.encode(answer):
            if on_token is not None:
                on_token(t)
        return {"id": "x", "object": "chat.completion", "created": 0, "model": "m",
                "choices": [{"index": 0, "message": {"role": "assistant", "content": answer}, "finish_reason": "length"}],
                "usage": {"prompt_tokens": 1, "completion_tokens": len(answer), "total_tokens": 1 + len(answer)}}

    srv._chat_completions = fake
    c = TestClient(create_app(srv))
    base = {"messages": [{"role": "user", "content": "hi"}]}
    cut = c.post("/v1/chat/completions", json={**base, "stop": ["END", "never"]}).json()["choices"][0]
    assert cut["message"]["content"] == "The arm lifts the cube. " and cut["finish_reason"] == "stop"
    same = c.post("/v1/chat/completions", json={**base, "stop": "never"}).json()["choices"][0]
    assert same["message"]["content"] == answer and same["finish_reason"] == "length"
    for stop, want in (("END", "The arm lifts the cube. "), ("ENX", answer), (None, answer)):
        pieces, finish = [], None
        with c.stream("POST", "/v1/chat/completions", json={**base, "stream": True, **({"stop": stop} if stop else {})}) as s:
            for line in s.iter_lines():
                if line.startswith("data: ") and line != "data: [DONE]":
                    ch = json.loads(line[6:])["choices"][0]
                    pieces.append(ch["delta"].get("content") or "")
                    finish = ch["finish_reason"] or finish
        assert "".join(pieces) == want, (stop, "".join(pieces))
        assert finish == ("stop" if stop == "END" else "length")


def test_metrics_as_json_and_in_the_prometheus_text_format(client):
    client.post("/v1/chat/completions", json={"max_tokens": 2, "temperature": 0.0, "messages": [{"role": "user", "content": "hi"}]})
    js = client.get("/metrics").json()
    assert js["requests"] >= 1
    txt = client.get("/metrics?format=prometheus")
    assert txt.status_code == 200 and txt.headers["content-type"].startswith("text/plain")
    lines = txt.text.splitlines()
    assert "# TYPE cosmos_b200_requests gauge" in lines
    val = [ln for ln in lines if ln.startswith("cosmos_b200_requests ")][0].split()[1]
    assert float(val) >= 1
    assert client.get("/metrics", headers={"accept": "text/plain"}).text.startswith("# TYPE")

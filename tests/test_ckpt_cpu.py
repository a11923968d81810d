"""Checkpoint IO: sharded save / load round trip, range reads for parameter shards, training state,
and corrupted files (truncated data, truncated header, header that lies about a tensor)."""
import json
import struct

import pytest
import torch

from cosmos_b200.ckpt import safetensors_io as sio


def _model():
    from cosmos_b200.config import tiny_config
    from cosmos_b200.models.mot import MoTModel

    m = MoTModel(tiny_config(n_layers=2), dtype=torch.float32, device="cpu")
    m.init_weights(seed=5)
    return m


def test_model_roundtrip_sharded_and_single(tmp_path):
    m = _model()
    sio.save_model(m, tmp_path / "sharded", max_shard_bytes=1 << 20)   # forces several shard files + index
    sio.save_model(m, tmp_path / "single")
    assert (tmp_path / "sharded" / sio.INDEX_NAME).exists() and (tmp_path / "single" / "model.safetensors").exists()
    want = {k: v.detach().clone() for k, v in sio.model_state(m).items()}
    for d in ("sharded", "single"):
        m2 = _model()
        with torch.no_grad():
            for p in m2.parameters():
                p.zero_()
        missing = sio.load_model(m2, tmp_path / d)
        assert not list(missing)
        got = sio.model_state(m2)
        assert all(torch.equal(got[k], want[k]) for k in want)


def test_range_read_gives_a_parameter_shard(tmp_path):
    m = _model()
    sio.save_model(m, tmp_path / "ck")
    name, full = next((k, v) for k, v in sio.model_state(m).items() if v.numel() >= 4096)
    flat = full.detach().reshape(-1)
    world = 4
    n = flat.numel() // world
    for r in range(world):
        dst = torch.empty(n, dtype=torch.bfloat16)          # converted on the way, as a bf16 shard would be
        sio.read_range(tmp_path / "ck", name, dst, r * n)
        assert torch.equal(dst, flat[r * n:(r + 1) * n].bfloat16())
    with pytest.raises(RuntimeError):
        sio.read_range(tmp_path / "ck", name, torch.empty(n + 1), (world - 1) * n + 1)


def test_train_state_roundtrip(tmp_path):
    t = {"m": torch.randn(10), "v": torch.rand(10), "i": torch.arange(5)}
    torch.manual_seed(1234)
    sio.save_train_state(tmp_path / "rank0.safetensors", 17, t, {"lr": 1e-4})
    a = torch.rand(3)
    step, got, extra = sio.load_train_state(tmp_path / "rank0.safetensors")
    b = torch.rand(3)                       # the RNG state travelled with the checkpoint
    assert step == 17 and extra == {"lr": 1e-4} and torch.equal(a, b)
    assert all(torch.equal(got[k], t[k]) for k in t)
    assert not (tmp_path / "rank0.safetensors.tmp").exists()


def _corrupt(path, how):
    raw = path.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    if how == "truncated_data":
        path.write_bytes(raw[:-64])
    elif how == "truncated_header":
        path.write_bytes(raw[:8 + n // 2])
    elif how == "lying_offsets":
        hdr = json.loads(raw[8:8 + n])
        k = next(k for k in hdr if k != "__metadata__")
        hdr[k]["data_offsets"][1] += 4
        h = json.dumps(hdr).encode()
        path.write_bytes(struct.pack("<Q", len(h)) + h + raw[8 + n:])
    elif how == "not_json":
        path.write_bytes(raw[:8] + b"\x00" * n + raw[8 + n:])


@pytest.mark.parametrize("how", ["truncated_data", "truncated_header", "lying_offsets", "not_json"])
def test_corrupted_checkpoint_is_rejected_with_a_message(tmp_path, how):
    m = _model()
    sio.save_model(m, tmp_path / "ck")
    _corrupt(tmp_path / "ck" / "model.safetensors", how)
    with pytest.raises(Exception) as ei:
        sio.load_model(_model(), tmp_path / "ck")
    msg = str(ei.value)
    assert any(w in msg.lower() for w in ("truncated", "safetensors", "bytes", "json", "header", "deserializ")), msg


def test_checkpoint_name_resolves_through_the_local_hub_cache(tmp_path, monkeypatch):
    """`--checkpoint-path Cosmos3-Nano` means the repo `nvidia/Cosmos3-Nano`; it is looked up in the local hub
    cache only, and the revision named by refs/main wins over other snapshots."""
    import torch
    from cosmos_b200.ckpt.resolve import repo_id, resolve_checkpoint_dir
    from cosmos_b200.pipeline import Cosmos3OmniPipeline
    assert repo_id("Cosmos3-Nano") == "nvidia/Cosmos3-Nano" and repo_id("acme/My-Model") == "acme/My-Model"
    monkeypatch.setenv("HF_HOME", str(tmp_path / "hf"))
    monkeypatch.delenv("HF_HUB_CACHE", raising=False)
    assert resolve_checkpoint_dir("Cosmos3-Nano") is None
    pipe = Cosmos3OmniPipeline.from_pretrained("tiny", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16),
                                               config_overrides=dict(n_layers=1, max_text_len=16), seed=5)
    base = tmp_path / "hf" / "hub" / "models--nvidia--Cosmos3-Nano"
    (base / "snapshots" / "stale").mkdir(parents=True)          # a snapshot without components is skipped
    snap = base / "snapshots" / "abc123"
    pipe.save_pretrained(snap)
    (base / "refs").mkdir()
    (base / "refs" / "main").write_text("abc123\n")
    assert resolve_checkpoint_dir("Cosmos3-Nano") == snap
    assert resolve_checkpoint_dir("nvidia/Cosmos3-Nano") == snap
    assert resolve_checkpoint_dir(str(snap)) == snap and resolve_checkpoint_dir(str(tmp_path)) is None
    again = Cosmos3OmniPipeline.from_pretrained("Cosmos3-Nano", torch_dtype=torch.float32, vae_widths=(8, 16, 16, 16), seed=9)
    assert again.cfg.n_layers == 1 and again.cfg.max_text_len == 16      # the stored config, not the 16B one
    a, b = pipe.transformer.state_dict(), again.transformer.state_dict()
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)

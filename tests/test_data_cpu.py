"""Training data pipeline (data/video_text.py): dataset, sharded resumable sampler, ordered prefetch, latent batches,
and the training CLI fed from a folder of clips."""
import json
import time

import numpy as np
import pytest
import torch

from cosmos_b200.data.video_text import LatentBatcher, Prefetcher, ShardedSampler, VideoTextDataset
from cosmos_b200.models.vae import CausalVideoVAE
from cosmos_b200.utils.tokenizer import load_tokenizer


def _make_dataset(root, n=7):
    rng = np.random.default_rng(0)
    for i in range(n):
        frames = (rng.random((6 + i, 40, 56, 3)) * 255).astype(np.uint8)
        frames[:, 0, 0, 0] = i                                   # marks the clip
        sub = root / ("a" if i % 2 else "b")
        sub.mkdir(exist_ok=True)
        np.savez(sub / f"clip{i}.npz", frames=frames, fps=12.0)
        if i % 3 == 0:
            (sub / f"clip{i}.json").write_text(json.dumps({"temporal_caption": f"clip {i}", "fps": 12}))
        else:
            (sub / f"clip{i}.txt").write_text(f"caption of clip {i}\n")
    (root / "orphan.npy").write_bytes(b"")                       # no caption beside it: not an item


def test_dataset_items_are_cut_padded_resized_and_captioned(tmp_path):
    _make_dataset(tmp_path)
    ds = VideoTextDataset(tmp_path, num_frames=9, width=32, height=32)
    assert len(ds) == 7
    names = [ds[i]["name"] for i in range(len(ds))]
    assert names == sorted(names) and "orphan.npy" not in names
    it = ds[names.index("b/clip0.npz")]
    assert it["video"].shape == (9, 32, 32, 3) and it["video"].dtype == np.uint8
    assert (it["video"][6:] == it["video"][5]).all()             # 6 source frames: the last one is repeated
    assert json.loads(it["caption"]) == {"temporal_caption": "clip 0", "fps": 12} and "\n" not in it["caption"]
    assert ds[names.index("a/clip1.npz")]["caption"] == "caption of clip 1"
    half = VideoTextDataset(tmp_path, num_frames=5, width=56, height=40, fps=6.0)    # 12 -> 6 fps: every other frame
    full = VideoTextDataset(tmp_path, num_frames=12, width=56, height=40)
    k = names.index("a/clip5.npz")
    assert np.array_equal(half[k]["video"][:5], full[k]["video"][0:10:2]) and half[k]["fps"] == 6.0
    with pytest.raises(FileNotFoundError):
        VideoTextDataset(tmp_path / "missing", 5, 8, 8)
    (tmp_path / "empty").mkdir()
    with pytest.raises(ValueError, match="no captioned clips"):
        VideoTextDataset(tmp_path / "empty", 5, 8, 8)


def test_index_file_lists_the_items(tmp_path):
    _make_dataset(tmp_path, 3)
    (tmp_path / "index.jsonl").write_text(json.dumps({"video": "b/clip0.npz", "caption": {"temporal_caption": "x"}}) + "\n\n"
                                          + json.dumps({"video": "a/clip1.npz", "caption": "plain"}) + "\n")
    ds = VideoTextDataset(tmp_path, 5, 16, 16)
    assert len(ds) == 2 and ds[0]["caption"] == '{"temporal_caption":"x"}' and ds[1]["caption"] == "plain"
    (tmp_path / "index.jsonl").write_text('{"video": "a/clip1.npz"}\n')
    with pytest.raises(ValueError, match="needs 'video' and 'caption'"):
        VideoTextDataset(tmp_path, 5, 16, 16)


def test_sampler_shards_without_overlap_and_resumes():
    n, world = 23, 4
    streams = []
    for r in range(world):
        it = iter(ShardedSampler(n, r, world, seed=3))
        streams.append([next(it) for _ in range(2 * (n // world))])
    first = [s[:n // world] for s in streams]
    flat = [i for s in first for i in s]
    assert len(set(flat)) == len(flat) == world * (n // world)          # one epoch: disjoint shards
    assert first[0] != streams[0][n // world:]                          # the next epoch is another permutation
    a = ShardedSampler(n, 1, world, seed=3)
    ita = iter(a)
    head = [next(ita) for _ in range(7)]
    state = a.state_dict()
    tail = [next(ita) for _ in range(9)]
    b = ShardedSampler(n, 1, world, seed=99)
    b.load_state_dict(state)
    itb = iter(b)
    assert [next(itb) for _ in range(9)] == tail and (head + tail)[:10] == streams[1]
    with pytest.raises(ValueError):
        ShardedSampler(n + 1, 1, world).load_state_dict(state)
    with pytest.raises(ValueError):
        ShardedSampler(2, 0, 4)


def test_prefetcher_keeps_order_reports_errors_and_gives_resume_points(tmp_path):
    _make_dataset(tmp_path)
    ds = VideoTextDataset(tmp_path, 5, 16, 16)
    slow = ds.__class__.__getitem__

    class Jittery(VideoTextDataset):
        def __getitem__(self, i):
            time.sleep(0.002 * ((i * 7) % 5))                           # items finish out of order
            return slow(self, i)

    jd = Jittery(tmp_path, 5, 16, 16)
    want = iter(ShardedSampler(len(ds), 0, 1, seed=5))
    pf = Prefetcher(jd, ShardedSampler(len(ds), 0, 1, seed=5), batch_size=2, depth=3, workers=3)
    states = []
    for _ in range(6):
        batch = next(pf)
        assert [s["name"] for s in batch] == [ds[next(want)]["name"] for _ in range(2)]
        states.append(pf.resume_state)
    pf.close()
    # resuming from the state taken after batch 3 continues with batch 4
    s2 = ShardedSampler(len(ds), 0, 1, seed=5)
    s2.load_state_dict(states[2])
    pf2 = Prefetcher(ds, s2, batch_size=2, depth=2, workers=1)
    ref = iter(ShardedSampler(len(ds), 0, 1, seed=5))
    for _ in range(6):
        next(ref)
    assert [s["name"] for s in next(pf2)] == [ds[next(ref)]["name"] for _ in range(2)]
    pf2.close()

    class Broken(VideoTextDataset):
        def __getitem__(self, i):
            raise OSError("disk gone")

    pf3 = Prefetcher(Broken(tmp_path, 5, 16, 16), ShardedSampler(len(ds), 0, 1), batch_size=1)
    with pytest.raises(OSError, match="disk gone"):
        next(pf3)
    pf3.close()


def test_latent_batcher_shapes_and_text_ids(tmp_path):
    _make_dataset(tmp_path, 3)
    ds = VideoTextDataset(tmp_path, 9, 32, 32)
    vae = CausalVideoVAE(16, (8, 16, 16, 16)).eval()
    tok = load_tokenizer(None, 512)
    lb = LatentBatcher(vae, tok, text_len=12, vocab_size=512, device="cpu", dtype=torch.float32)
    lat, ids = lb([ds[0], ds[1]])
    assert lat.shape == (2, 16, 3, 4, 4) and ids.shape == (2, 12) and ids.dtype == torch.long
    assert int(ids.max()) < 512 and torch.isfinite(lat).all()
    x = CausalVideoVAE.from_uint8(torch.from_numpy(np.stack([ds[0]["video"], ds[1]["video"]])))
    assert torch.allclose(lat, vae.encode(x, chunk_frames=4), atol=1e-5)


def test_training_cli_reads_clips_and_resumes_its_data_stream(tmp_path, capsys):
    from cosmos_b200 import train
    data = tmp_path / "data"
    data.mkdir()
    _make_dataset(data, 6)
    save = tmp_path / "ckpt"
    common = ["--model", "tiny", "--layers", "1", "--latent", "16,2,4,4", "--text-len", "8", "--data-root", str(data),
              "--vae-widths", "8,16,16,16", "--save-dir", str(save), "--warmup", "0", "--data-workers", "1"]
    assert train.main(common + ["--steps", "2"]) == 0
    first = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert [r["step"] for r in first if "step" in r] == [1, 2] and all(np.isfinite(r["loss"]) for r in first if "loss" in r)
    state = json.loads((save / "data_state_rank00000.json").read_text())
    assert state["offset"] == 2 and state["epoch"] == 0
    assert train.main(common + ["--steps", "1", "--resume"]) == 0
    out = [json.loads(line) for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert [r["step"] for r in out if "step" in r] == [3]
    assert json.loads((save / "data_state_rank00000.json").read_text())["offset"] == 3

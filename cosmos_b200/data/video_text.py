"""Training data: captioned video clips -> (latents, text ids) batches.

The reference points to a training guide outside its tree (README.md:653-655) and shows its data side only through
the action cookbook's dataset items (`video [C,T,H,W] uint8`, `ai_caption`, `conditioning_fps`; reference
cookbooks/cosmos3/generator/action/run_fd_with_cosmos_framework.ipynb:750-790). This module is the general
form of that: a folder of clips with sidecar captions, sharded over the data-parallel ranks, decoded and resized on
host threads while the GPU trains, encoded by the tokenizer VAE on the device.

Layout of a dataset folder (searched recursively): every media file `<stem>.{mp4,npy,npz,png,jpg,jpeg}` with a caption
beside it in `<stem>.json` (a structured prompt, fed as compact JSON, see io/prompt_schema.py) or `<stem>.txt`.
Alternatively an index file `index.jsonl` with one `{"video": relative path, "caption": str | object}` per line.

Pieces:
* `VideoTextDataset` - map-style; an item is {"video" uint8 [T, H, W, 3], "caption", "fps", "name"}; clips are resampled
  to the requested frame rate, cut or padded (last frame repeated) to the requested length, resized with a centre crop.
* `ShardedSampler` - a seeded permutation per epoch, split across data ranks without overlap; resumable.
* `Prefetcher` - host threads that prepare the next batches (decode + resize) ahead of the consumer, in order.
* `LatentBatcher` - pinned staging buffer -> device copy -> VAE encode (no grad) and caption -> token ids.
"""
from __future__ import annotations

import json
import queue
import threading
from pathlib import Path
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..io import media

MEDIA_SUFFIXES = (".mp4", ".npy", ".npz", ".png", ".jpg", ".jpeg")


def _caption_text(value: Any) -> str:
    if isinstance(value, (dict, list)):
        return json.dumps(value, separators=(",", ":"), ensure_ascii=False)
    return str(value).strip()


class VideoTextDataset:
    def __init__(self, root, num_frames: int, width: int, height: int, fps: Optional[float] = None):
        """`num_frames` pixel frames per item at `width` x `height`; `fps` resamples clips in time (None keeps
        every source frame)."""
        self.root = Path(root)
        if not self.root.is_dir():
            raise FileNotFoundError(f"dataset folder {self.root} does not exist")
        self.num_frames, self.size, self.fps = int(num_frames), (int(width), int(height)), fps
        self.items: List[Tuple[Path, Any]] = []
        index = self.root / "index.jsonl"
        if index.exists():
            for n, line in enumerate(index.read_text().splitlines()):
                if not line.strip():
                    continue
                row = json.loads(line)
                if "video" not in row or "caption" not in row:
                    raise ValueError(f"{index}:{n + 1}: a row needs 'video' and 'caption'")
                self.items.append((self.root / row["video"], row["caption"]))
        else:
            for p in sorted(self.root.rglob("*")):
                if p.suffix.lower() not in MEDIA_SUFFIXES or not p.is_file():
                    continue
                for cap in (p.with_suffix(".json"), p.with_suffix(".txt")):
                    if cap.exists():
                        self.items.append((p, cap))
                        break
        if not self.items:
            raise ValueError(f"no captioned clips under {self.root}")

    def __len__(self) -> int:
        return len(self.items)

    def caption(self, i: int) -> str:
        cap = self.items[i][1]
        if isinstance(cap, Path):
            text = cap.read_text()
            if cap.suffix == ".json":
                try:
                    return _caption_text(json.loads(text))
                except json.JSONDecodeError as e:
                    raise ValueError(f"{cap} is not valid JSON: {e}") from e
            return text.strip()
        return _caption_text(cap)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        path = self.items[i][0]
        frames, src_fps = media.read_video(path)
        if self.fps and src_fps and frames.shape[0] > 1:
            # nearest source frame for every target time stamp
            n_out = max(1, int(round(frames.shape[0] * float(self.fps) / float(src_fps))))
            idx = np.minimum(np.round(np.arange(n_out) * float(src_fps) / float(self.fps)).astype(np.int64),
                             frames.shape[0] - 1)
            frames = frames[idx]
        frames = frames[:self.num_frames]
        if (frames.shape[2], frames.shape[1]) != self.size:
            from PIL import Image
            frames = np.stack([np.asarray(media._resize_center_crop(Image.fromarray(f), self.size)) for f in frames])
        if frames.shape[0] < self.num_frames:
            frames = np.concatenate([frames, np.repeat(frames[-1:], self.num_frames - frames.shape[0], axis=0)])
        return {"video": np.ascontiguousarray(frames), "caption": self.caption(i), "fps": float(self.fps or src_fps),
                "name": str(path.relative_to(self.root))}


class ShardedSampler:
    """Index stream for one data-parallel rank: epoch e visits a permutation seeded by (seed, e); rank r takes
    positions r, r + world, ... of it (the tail that does not fill every rank is dropped, so all ranks take the
    same number of steps). `state_dict()` after k draws resumes at draw k + 1."""

    def __init__(self, n: int, rank: int = 0, world: int = 1, seed: int = 0, shuffle: bool = True):
        if n < world:
            raise ValueError(f"{n} samples cannot feed {world} data ranks")
        self.n, self.rank, self.world, self.seed, self.shuffle = n, rank, world, seed, shuffle
        self.epoch, self.offset = 0, 0
        self.per_rank = n // world

    def _order(self, epoch: int) -> np.ndarray:
        if not self.shuffle:
            return np.arange(self.n)
        return np.random.default_rng([self.seed, epoch]).permutation(self.n)

    def __iter__(self) -> Iterator[int]:
        while True:
            order = self._order(self.epoch)
            while self.offset < self.per_rank:
                i = int(order[self.offset * self.world + self.rank])
                self.offset += 1
                yield i
            self.epoch, self.offset = self.epoch + 1, 0

    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "offset": self.offset, "seed": self.seed, "n": self.n, "world": self.world}

    def load_state_dict(self, s: Dict[str, int]) -> None:
        if int(s["n"]) != self.n or int(s["world"]) != self.world:
            raise ValueError("sampler state belongs to another dataset size or data-parallel degree")
        self.epoch, self.offset, self.seed = int(s["epoch"]), int(s["offset"]), int(s["seed"])


class Prefetcher:
    """Prepares batches on host threads ahead of the consumer. Batches come out in sampler order whatever the
    thread timing; an exception in a worker is raised by the `next()` that would have returned its batch."""

    def __init__(self, dataset: VideoTextDataset, sampler: ShardedSampler, batch_size: int, depth: int = 2,
                 workers: int = 2):
        self.dataset, self.batch_size, self.depth = dataset, batch_size, max(1, depth)
        self._it = iter(sampler)
        self._sampler = sampler
        self._todo: "queue.Queue" = queue.Queue()
        self._done: Dict[int, Any] = {}
        self._cv = threading.Condition()
        self._next_submit = self._next_take = 0
        self._states: Dict[int, Dict[str, int]] = {}
        self._closed = False
        self._threads = [threading.Thread(target=self._work, daemon=True) for _ in range(max(1, workers))]
        for t in self._threads:
            t.start()
        for _ in range(self.depth):
            self._submit()

    def _submit(self) -> None:
        idx = [next(self._it) for _ in range(self.batch_size)]
        self._states[self._next_submit] = self._sampler.state_dict()   # sampler state AFTER this batch was drawn
        self._todo.put((self._next_submit, idx))
        self._next_submit += 1

    def _work(self) -> None:
        while True:
            job = self._todo.get()
            if job is None:
                return
            k, idx = job
            try:
                out: Any = [self.dataset[i] for i in idx]
            except BaseException as e:  # noqa: BLE001 - handed to the consumer
                out = e
            with self._cv:
                self._done[k] = out
                self._cv.notify_all()

    def __iter__(self):
        return self

    def __next__(self) -> List[Dict[str, Any]]:
        if self._closed:
            raise StopIteration
        k = self._next_take
        with self._cv:
            while k not in self._done:
                self._cv.wait(0.1)
            out = self._done.pop(k)
        self._next_take += 1
        self.resume_state = self._states.pop(k)    # resuming from here continues with batch k + 1
        self._submit()
        if isinstance(out, BaseException):
            raise out
        return out

    def close(self) -> None:
        self._closed = True
        for _ in self._threads:
            self._todo.put(None)


class LatentBatcher:
    """Host samples -> device tensors for `Trainer.train_step`: frames go through one pinned staging buffer to the
    device (asynchronous copy on CUDA), the VAE encodes them without gradients, captions become padded token ids."""

    def __init__(self, vae, tokenizer, text_len: int, vocab_size: int, device, dtype):
        self.vae, self.tokenizer, self.text_len, self.vocab_size = vae, tokenizer, text_len, vocab_size
        self.device, self.dtype = torch.device(device), dtype
        self._stage: Optional[torch.Tensor] = None

    def text_ids(self, captions: Sequence[str]) -> torch.Tensor:
        rows = []
        for c in captions:
            ids = list(self.tokenizer.encode(c))
            pad = getattr(self.tokenizer, "pad_id", 0) or 0
            ids = (ids + [pad] * self.text_len)[:self.text_len]
            rows.append([min(int(t), self.vocab_size - 1) for t in ids])
        return torch.tensor(rows, dtype=torch.long)

    @torch.no_grad()
    def __call__(self, samples: Sequence[Dict[str, Any]]) -> Tuple[torch.Tensor, torch.Tensor]:
        from ..models.vae import CausalVideoVAE
        video = np.stack([s["video"] for s in samples])                       # [B, T, H, W, 3] uint8
        if self._stage is None or self._stage.shape != video.shape:
            self._stage = torch.empty(video.shape, dtype=torch.uint8, pin_memory=self.device.type == "cuda")
        self._stage.copy_(torch.from_numpy(video))
        frames = self._stage.to(self.device, non_blocking=True)
        x = CausalVideoVAE.from_uint8(frames).to(self.dtype)                  # [B, 3, T, H, W] in [-1, 1]
        latents = self.vae.encode(x, chunk_frames=4 if x.shape[2] > 1 else None).to(self.dtype)
        ids = self.text_ids([s["caption"] for s in samples]).to(self.device, non_blocking=True)
        return latents, ids

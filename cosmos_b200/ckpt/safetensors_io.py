"""Safetensors checkpoints: single file or sharded with `model.safetensors.index.json`
(the Hugging Face layout the reference's checkpoints use; reference README.md:214,242-246),
in a Diffusers-style component layout:

    <root>/model_index.json
    <root>/transformer/{config.json, model-0000x-of-0000N.safetensors, model.safetensors.index.json}
    <root>/vae/{config.json, model.safetensors}
    <root>/sound_tokenizer/{config.json, model.safetensors}
    <root>/scheduler/scheduler_config.json

Loading goes through the package's own memory-mapped reader (C++, `csrc/safetensors_reader.cpp`:
every offset of the header is validated against the file before a byte is copied, and a tensor or
any element range of it is copied straight from the mapping into the destination, CPU or CUDA), so
a rank reads only what it needs, e.g. its shard of a flat parameter (`read_range`). Without the
built extension the `safetensors` package's `safe_open` is used. Training state (optimizer shards,
RNG, step) is saved per rank with an atomic rename.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Callable, Dict, Iterable, Optional

import torch
from safetensors import safe_open
from safetensors.torch import save_file

INDEX_NAME = "model.safetensors.index.json"


def save_sharded(state: Dict[str, torch.Tensor], out_dir, max_shard_bytes: int = 5 << 30,
                 metadata: Optional[Dict[str, str]] = None) -> None:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    shards, cur, cur_bytes = [], {}, 0
    for k, v in state.items():
        nb = v.numel() * v.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v.detach().contiguous().cpu()
        cur_bytes += nb
    if cur:
        shards.append(cur)
    if len(shards) == 1:
        _atomic_save(shards[0], out_dir / "model.safetensors", metadata)
        return
    weight_map, total = {}, 0
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        _atomic_save(sh, out_dir / name, metadata)
        for k, v in sh.items():
            weight_map[k] = name
            total += v.numel() * v.element_size()
    tmp = out_dir / (INDEX_NAME + ".tmp")
    tmp.write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=1))
    os.replace(tmp, out_dir / INDEX_NAME)


def _atomic_save(tensors, path: Path, metadata=None) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    save_file(tensors, str(tmp), metadata=metadata or {"format": "pt"})
    os.replace(tmp, path)


class _PyReader:
    """`safe_open`-based stand-in with the interface of the native `SafetensorsFile`."""

    def __init__(self, path: str):
        self._f = safe_open(path, "pt")
        self._meta = self._f.metadata() or {}

    def keys(self):
        return list(self._f.keys())

    def has(self, name):
        return name in self._f.keys()

    def shape(self, name):
        return list(self._f.get_slice(name).get_shape())

    def get(self, name):
        return self._f.get_tensor(name)

    def metadata(self, key):
        return self._meta.get(key, "")

    def metadata_keys(self):
        return sorted(self._meta)

    def read_into(self, name, dst, elem_offset):
        src = self._f.get_tensor(name).reshape(-1)[elem_offset:elem_offset + dst.numel()]
        dst.view(-1).copy_(src)


def open_reader(path):
    """Reader for one .safetensors file: the native memory-mapped one when the extension is built."""
    from .. import ops

    if ops.load_extension(build_if_missing=False):
        return torch.classes.cosmos_b200.SafetensorsFile(str(path))
    return _PyReader(str(path))


def read_range(model_dir, name: str, dst: torch.Tensor, elem_offset: int = 0) -> None:
    """Fills `dst` (contiguous, any device) with elements [elem_offset, elem_offset + dst.numel()) of the
    flattened checkpoint tensor `name`: a rank's shard of a parameter without touching the rest."""
    files = tensor_files(model_dir)
    if name not in files:
        raise KeyError(f"checkpoint has no tensor {name}")
    open_reader(files[name]).read_into(name, dst, int(elem_offset))


def tensor_files(model_dir) -> Dict[str, Path]:
    """tensor name -> file that holds it."""
    model_dir = Path(model_dir)
    idx = model_dir / INDEX_NAME
    if idx.exists():
        wm = json.loads(idx.read_text())["weight_map"]
        return {k: model_dir / v for k, v in wm.items()}
    single = model_dir / "model.safetensors"
    if not single.exists():
        raise FileNotFoundError(f"no safetensors checkpoint under {model_dir}")
    return {k: single for k in open_reader(single).keys()}


def load_into(model_dir, targets: Dict[str, torch.Tensor], strict: bool = True,
              slicer: Optional[Callable[[str, "object"], torch.Tensor]] = None) -> Iterable[str]:
    """Copies checkpoint tensors into `targets` (name -> destination tensor, any device/dtype).
    `slicer(name, safetensors_slice)` may return only a part of a tensor (TP / FSDP shard reads)."""
    files = tensor_files(model_dir)
    missing = [k for k in targets if k not in files]
    if strict and missing:
        raise KeyError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:3]}")
    by_file: Dict[Path, list] = {}
    for k in targets:
        if k in files:
            by_file.setdefault(files[k], []).append(k)
    with torch.no_grad():
        for path, names in by_file.items():
            if slicer is not None:
                with safe_open(str(path), "pt") as f:
                    for k in names:
                        src = slicer(k, f.get_slice(k))
                        dst = targets[k]
                        if tuple(src.shape) != tuple(dst.shape):
                            raise ValueError(f"{k}: checkpoint shape {tuple(src.shape)} != model {tuple(dst.shape)}")
                        dst.copy_(src.to(dst.dtype))
                continue
            f = open_reader(path)
            for k in names:
                dst = targets[k]
                shape = tuple(f.shape(k))
                if shape != tuple(dst.shape):
                    raise ValueError(f"{k}: checkpoint shape {shape} != model {tuple(dst.shape)}")
                if dst.is_contiguous():
                    f.read_into(k, dst, 0)  # straight from the mapping into the parameter storage
                else:
                    dst.copy_(f.get(k).to(dst.dtype))
    return missing


def model_state(model) -> Dict[str, torch.Tensor]:
    """Named tensors of a MoTModel with per-layer flat buffers expanded to their named views
    (`dm.layers.3.wqkv`, ...), which is the on-disk naming."""
    from ..models.mot import FlatLayer

    out: Dict[str, torch.Tensor] = {}
    flat_prefixes = []
    for mod_name, mod in model.named_modules():
        if isinstance(mod, FlatLayer):
            flat_prefixes.append(mod_name + ".flat")
            for k, v in mod.views().items():
                out[f"{mod_name}.{k}"] = v
    for name, p in model.named_parameters():
        if name not in flat_prefixes:
            out[name] = p
    return out


def save_model(model, out_dir, max_shard_bytes: int = 5 << 30) -> None:
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    save_sharded({k: v.detach() for k, v in model_state(model).items()}, out_dir, max_shard_bytes)
    if hasattr(model, "cfg"):
        (out_dir / "config.json").write_text(json.dumps(model.cfg.to_dict(), indent=1))


def load_model(model, model_dir, strict: bool = True):
    return load_into(model_dir, {k: v.data for k, v in model_state(model).items()}, strict)


def save_train_state(path, step: int, tensors: Dict[str, torch.Tensor], extra: Optional[dict] = None) -> None:
    """Per-rank training state (optimizer shards etc.) + step + RNG, written atomically."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    meta = {"step": str(step), "extra": json.dumps(extra or {})}
    t = {k: v.detach().contiguous().cpu() for k, v in tensors.items()}
    t["__rng_cpu"] = torch.get_rng_state()
    _atomic_save(t, path, meta)


def load_train_state(path):
    f = open_reader(path)
    meta = {k: f.metadata(k) for k in f.metadata_keys()}
    tensors = {k: f.get(k) for k in f.keys()}
    rng = tensors.pop("__rng_cpu", None)
    if rng is not None:
        torch.set_rng_state(rng)
    return int(meta["step"]), tensors, json.loads(meta.get("extra", "{}"))

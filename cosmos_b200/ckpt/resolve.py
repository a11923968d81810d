"""Where a checkpoint name points on this machine.

`--checkpoint-path` / `from_pretrained` take a directory or a model name; a bare name is a Hugging Face repo
id under `nvidia/` (reference cookbooks/cosmos3/generator/audiovisual/README.md:60,64). Names are looked up
in the local hub cache only (`HF_HUB_CACHE`, else `$HF_HOME/hub`, else `~/.cache/huggingface/hub`; layout
`models--<org>--<repo>/snapshots/<revision>/`, revision from `refs/main` when present): nothing is downloaded.
A name with no local snapshot resolves to None and the caller builds the architecture with random weights."""
from __future__ import annotations

import os
from pathlib import Path
from typing import List, Optional

COMPONENT_DIR = "transformer"  # a checkpoint directory is recognised by this component folder


def hub_cache_dirs() -> List[Path]:
    out = []
    if os.environ.get("HF_HUB_CACHE"):
        out.append(Path(os.environ["HF_HUB_CACHE"]))
    if os.environ.get("HF_HOME"):
        out.append(Path(os.environ["HF_HOME"]) / "hub")
    out.append(Path.home() / ".cache" / "huggingface" / "hub")
    return out


def repo_id(name: str) -> str:
    name = name.strip("/")
    return name if "/" in name else f"nvidia/{name}"


def resolve_checkpoint_dir(name_or_path: str) -> Optional[Path]:
    """Directory that holds `transformer/` (and optionally `vae/`, `sound_tokenizer/`, `scheduler/`), or None."""
    path = Path(name_or_path)
    if path.is_dir():
        return path if (path / COMPONENT_DIR).is_dir() else None
    org, _, repo = repo_id(str(name_or_path)).partition("/")
    for cache in hub_cache_dirs():
        base = cache / f"models--{org}--{repo}"
        snaps = base / "snapshots"
        if not snaps.is_dir():
            continue
        ref = base / "refs" / "main"
        cands = []
        if ref.is_file():
            cands.append(snaps / ref.read_text().strip())
        cands += sorted((p for p in snaps.iterdir() if p.is_dir()), key=lambda p: p.stat().st_mtime, reverse=True)
        for c in cands:
            if (c / COMPONENT_DIR).is_dir():
                return c
    return None

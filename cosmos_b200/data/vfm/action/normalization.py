"""Per-embodiment action normalisation.

Actions of different embodiments live on different scales (metres per frame of a car, centimetres of a gripper, a
0..1 gripper opening), so the action encoder sees them standardised per domain (`domain_name`: av, droid_lerobot,
umi, ...; reference cookbooks/cosmos3/generator/action/README.md:29-41, where the dataset readers are described as
normalising their actions). `ActionNormalizer` holds one (mean, std) pair per domain and action dimension, fitted on
a dataset or read from `action_stats.json` of a checkpoint; domains without statistics pass through unchanged. The
rot6d part of a pose is a rotation encoding, not a free vector, and stays as it is: only the dimensions listed in
`free_dims` (translation and gripper by default) are standardised."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable, Optional, Sequence

import numpy as np

STATS_FILE = "action_stats.json"


def default_free_dims(action_dim: int) -> Sequence[int]:
    """Translation (0..2) and everything after the 6 rot6d dimensions (gripper / hand joints)."""
    return [d for d in range(action_dim) if d < 3 or d >= 9]


class ActionNormalizer:
    def __init__(self, stats: Optional[Dict[str, Dict[str, list]]] = None, eps: float = 1e-6):
        """`stats[domain] = {"mean": [D], "std": [D], "free_dims": [...]}`."""
        self.stats = {k: {kk: list(vv) for kk, vv in v.items()} for k, v in (stats or {}).items()}
        self.eps = eps

    # ------------------------------------------------------------------ fitting / persistence
    def fit(self, domain: str, actions: Iterable[np.ndarray], free_dims: Optional[Sequence[int]] = None) -> None:
        """Statistics of a domain from chunks of actions [n_i, D]."""
        rows = np.concatenate([np.asarray(a, dtype=np.float64).reshape(-1, np.asarray(a).shape[-1]) for a in actions])
        if rows.shape[0] < 2:
            raise ValueError("at least two action rows are needed to fit statistics")
        self.stats[domain] = {"mean": rows.mean(0).tolist(), "std": rows.std(0).tolist(),
                              "free_dims": list(default_free_dims(rows.shape[1]) if free_dims is None else free_dims)}

    def save(self, directory) -> Path:
        path = Path(directory) / STATS_FILE
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(json.dumps(self.stats, indent=1))
        return path

    @classmethod
    def load(cls, directory) -> "ActionNormalizer":
        path = Path(directory) / STATS_FILE
        return cls(json.loads(path.read_text()) if path.exists() else None)

    # ------------------------------------------------------------------ use
    def _affine(self, domain: str, dim: int):
        st = self.stats.get(domain)
        if st is None:
            return None
        if len(st["mean"]) != dim:
            raise ValueError(f"statistics of '{domain}' are {len(st['mean'])}-D, the actions {dim}-D")
        mean, scale = np.zeros(dim), np.ones(dim)
        free = list(st.get("free_dims", default_free_dims(dim)))
        mean[free] = np.asarray(st["mean"])[free]
        scale[free] = np.maximum(np.asarray(st["std"])[free], self.eps)
        return mean, scale

    def normalize(self, actions, domain: str) -> np.ndarray:
        a = np.asarray(actions, dtype=np.float32)
        aff = self._affine(domain, a.shape[-1])
        return a if aff is None else ((a - aff[0]) / aff[1]).astype(np.float32)

    def denormalize(self, actions, domain: str) -> np.ndarray:
        a = np.asarray(actions, dtype=np.float32)
        aff = self._affine(domain, a.shape[-1])
        return a if aff is None else (a * aff[1] + aff[0]).astype(np.float32)

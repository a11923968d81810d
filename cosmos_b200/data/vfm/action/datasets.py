"""LeRobot v3.0 dataset reader for the DROID action domain.

Mirrors the reference's `cosmos_framework.data.vfm.action.datasets.DROIDLeRobotDataset` as used
in cookbooks/cosmos3/generator/action/run_fd_with_cosmos_framework.ipynb:750-790: `root` points
at a LeRobot v3 tree (`meta/info.json`, `data/chunk-*/file-*.parquet`, `videos/<camera>/...`);
item keys are `action [chunk, 10]`, `video [C, T, H, W] uint8`, `conditioning_fps`, `viewpoint`,
`ai_caption`. Actions are 10-D per transition: relative end-effector translation (3), rot6d (6),
gripper (1) (reference action/README.md:29-41). Video decoding uses this package's media reader (OpenCV's
bundled H.264 / AV1 decoders, else an ffmpeg binary), seeking to the item's first frame; on a host with neither,
items carry `video=None` and the rest of the sample (actions, caption, timing) is still served.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import pose_utils


def euler_xyz_to_matrix(e: np.ndarray) -> np.ndarray:
    """[..., 3] roll/pitch/yaw (extrinsic xyz) -> [..., 3, 3]."""
    x, y, z = e[..., 0], e[..., 1], e[..., 2]
    cx, sx, cy, sy, cz, sz = np.cos(x), np.sin(x), np.cos(y), np.sin(y), np.cos(z), np.sin(z)
    r = np.empty(e.shape[:-1] + (3, 3))
    r[..., 0, 0], r[..., 0, 1], r[..., 0, 2] = cz * cy, cz * sy * sx - sz * cx, cz * sy * cx + sz * sx
    r[..., 1, 0], r[..., 1, 1], r[..., 1, 2] = sz * cy, sz * sy * sx + cz * cx, sz * sy * cx - cz * sx
    r[..., 2, 0], r[..., 2, 1], r[..., 2, 2] = -sy, cy * sx, cy * cx
    return r


def cartesian_to_poses(cart: np.ndarray) -> np.ndarray:
    """[T, 6] (xyz + euler) -> [T, 4, 4]."""
    t = cart.shape[0]
    poses = np.tile(np.eye(4), (t, 1, 1))
    poses[:, :3, :3] = euler_xyz_to_matrix(cart[:, 3:6])
    poses[:, :3, 3] = cart[:, :3]
    return poses


class DROIDLeRobotDataset:
    def __init__(self, root, action_chunk_size: int = 16, cameras: Optional[Sequence[str]] = None,
                 state_key: str = "observation.state.cartesian_position",
                 gripper_key: str = "observation.state.gripper_position", stride: Optional[int] = None,
                 decode_video: bool = True):
        self.root = Path(root)
        self.info = json.loads((self.root / "meta" / "info.json").read_text())
        self.fps = int(self.info.get("fps", 15))
        self.chunk = action_chunk_size
        self.stride = stride or action_chunk_size
        self.decode_video = decode_video
        feats = self.info.get("features", {})
        self.cameras = list(cameras) if cameras else [k for k, v in feats.items() if v.get("dtype") == "video"]
        self.state_key, self.gripper_key = state_key, gripper_key
        import pandas as pd

        files = sorted((self.root / "data").glob("**/*.parquet"))
        if not files:
            raise FileNotFoundError(f"no parquet files under {self.root / 'data'}")
        self.frames = pd.concat([pd.read_parquet(f) for f in files], ignore_index=True)
        self.tasks = {}
        tpath = self.root / "meta" / "tasks.parquet"
        if tpath.exists():
            tdf = pd.read_parquet(tpath)
            for idx, row in tdf.iterrows():
                self.tasks[int(row.get("task_index", 0))] = str(idx) if "task" not in tdf.columns else str(row["task"])
        self.index: List[tuple] = []
        for ep, grp in self.frames.groupby("episode_index"):
            n = len(grp)
            for s in range(0, n - self.chunk, self.stride):
                self.index.append((int(ep), int(grp.index[0]) + s))

    def __len__(self) -> int:
        return len(self.index)

    def _column(self, rows, key: str) -> Optional[np.ndarray]:
        if key in rows.columns:
            return np.stack([np.asarray(v, dtype=np.float64) for v in rows[key].to_list()])
        return None

    def __getitem__(self, i: int) -> Dict:
        ep, start = self.index[i]
        rows = self.frames.iloc[start:start + self.chunk + 1]
        cart = self._column(rows, self.state_key)
        if cart is None:  # fall back to the first 6 dims of the flat state vector
            st = self._column(rows, "observation.state")
            cart = st[:, :6]
        grip = self._column(rows, self.gripper_key)
        grip = grip.reshape(len(rows), -1)[:, :1] if grip is not None else np.zeros((len(rows), 1))
        rel = pose_utils.pose_abs_to_rel(cartesian_to_poses(cart), "rot6d", "backward_framewise", 1.0)
        action = np.concatenate([rel, grip[1:]], axis=-1).astype(np.float32)  # [chunk, 10]
        video = None
        if self.decode_video and self.cameras:
            video = self._read_views(ep, rows)
        task_idx = int(rows["task_index"].iloc[0]) if "task_index" in rows.columns else 0
        return {"action": action, "video": video, "conditioning_fps": self.fps,
                "viewpoint": "+".join(c.split(".")[-1] for c in self.cameras) or "unknown",
                "ai_caption": self.tasks.get(task_idx, ""), "episode_index": ep,
                "frame_index": int(rows["frame_index"].iloc[0]) if "frame_index" in rows.columns else start}

    def _read_views(self, ep: int, rows) -> Optional[np.ndarray]:
        """Concatenates the camera views side by side: [C, T, H, W * n_views] uint8."""
        from ....io import media

        views = []
        t0 = int(rows["frame_index"].iloc[0]) if "frame_index" in rows.columns else 0
        for cam in self.cameras:
            files = sorted((self.root / "videos" / cam).glob("**/*.mp4"))
            if not files:
                continue
            try:
                frames, _ = media.read_video(files[0], max_frames=self.chunk + 1, start=t0)
            except Exception:  # noqa: BLE001 - codec not decodable on this host
                continue
            views.append(frames)
        if not views:
            return None
        n = min(v.shape[0] for v in views)
        vid = np.concatenate([v[:n] for v in views], axis=2)
        return np.ascontiguousarray(vid.transpose(3, 0, 1, 2))

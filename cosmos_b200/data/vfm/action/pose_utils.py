"""Camera/ego pose <-> relative action conversion.

API and conventions follow the reference's `cosmos_framework.data.vfm.action.pose_utils`
as used in cookbooks/cosmos3/generator/action/run_fd_with_cosmos_framework.ipynb:441-452,533 and
run_id_with_cosmos_framework.ipynb:588,661-670: poses are camera-to-world 4x4 matrices in the
OpenCV convention (x right, y down, z forward), metres; a relative action is 9-D =
translation (3) + the first two columns of the rotation matrix (rot6d, 6); the default
`pose_convention="backward_framewise"` expresses frame i+1 in the frame of i
(T_rel = inv(T_i) @ T_{i+1}); translations are divided by `translation_scale` (1.35 for the
AV domain, av_dataset.py constants quoted in run_id_with_cosmos_framework.ipynb:663).
"""
from __future__ import annotations

import numpy as np

ROTATION_FORMATS = ("rot6d",)
POSE_CONVENTIONS = ("backward_framewise", "backward_anchored")


def rotmat_to_rot6d(r: np.ndarray) -> np.ndarray:
    """[..., 3, 3] -> [..., 6]: first two columns, column-major (c0 then c1)."""
    return np.concatenate([r[..., :, 0], r[..., :, 1]], axis=-1)


def rot6d_to_rotmat(d6: np.ndarray) -> np.ndarray:
    """[..., 6] -> [..., 3, 3] by Gram-Schmidt; exact inverse of `rotmat_to_rot6d` on rotations."""
    a1, a2 = d6[..., :3], d6[..., 3:6]
    b1 = a1 / np.clip(np.linalg.norm(a1, axis=-1, keepdims=True), 1e-12, None)
    a2 = a2 - (b1 * a2).sum(-1, keepdims=True) * b1
    b2 = a2 / np.clip(np.linalg.norm(a2, axis=-1, keepdims=True), 1e-12, None)
    b3 = np.cross(b1, b2)
    return np.stack([b1, b2, b3], axis=-1)


def _inv_se3(t: np.ndarray) -> np.ndarray:
    r, p = t[..., :3, :3], t[..., :3, 3]
    out = np.zeros_like(t)
    rt = np.swapaxes(r, -1, -2)
    out[..., :3, :3] = rt
    out[..., :3, 3] = -(rt @ p[..., None])[..., 0]
    out[..., 3, 3] = 1.0
    return out


def pose_abs_to_rel(poses_abs: np.ndarray, rotation_format: str = "rot6d",
                    pose_convention: str = "backward_framewise", translation_scale: float = 1.0) -> np.ndarray:
    """poses_abs [T, 4, 4] -> actions [T-1, 9]."""
    poses_abs = np.asarray(poses_abs, dtype=np.float64)
    if poses_abs.ndim != 3 or poses_abs.shape[1:] != (4, 4):
        raise ValueError("poses_abs must be [T, 4, 4]")
    if rotation_format not in ROTATION_FORMATS:
        raise ValueError(f"rotation_format must be one of {ROTATION_FORMATS}")
    if pose_convention == "backward_framewise":
        rel = _inv_se3(poses_abs[:-1]) @ poses_abs[1:]
    elif pose_convention == "backward_anchored":
        rel = _inv_se3(poses_abs[:1]) @ poses_abs[1:]
    else:
        raise ValueError(f"pose_convention must be one of {POSE_CONVENTIONS}")
    trans = rel[:, :3, 3] / float(translation_scale)
    return np.concatenate([trans, rotmat_to_rot6d(rel[:, :3, :3])], axis=-1)


def pose_rel_to_abs(actions: np.ndarray, rotation_format: str = "rot6d",
                    pose_convention: str = "backward_framewise", translation_scale: float = 1.0,
                    initial_pose: np.ndarray = None) -> np.ndarray:
    """actions [T-1, 9] -> poses [T, 4, 4] starting from `initial_pose` (identity by default)."""
    actions = np.asarray(actions, dtype=np.float64)
    if actions.ndim != 2 or actions.shape[1] != 9:
        raise ValueError("actions must be [T-1, 9]")
    if rotation_format not in ROTATION_FORMATS:
        raise ValueError(f"rotation_format must be one of {ROTATION_FORMATS}")
    n = actions.shape[0]
    rel = np.tile(np.eye(4), (n, 1, 1))
    rel[:, :3, :3] = rot6d_to_rotmat(actions[:, 3:])
    rel[:, :3, 3] = actions[:, :3] * float(translation_scale)
    t0 = np.eye(4) if initial_pose is None else np.asarray(initial_pose, dtype=np.float64)
    out = [t0]
    for i in range(n):
        if pose_convention == "backward_framewise":
            out.append(out[-1] @ rel[i])
        elif pose_convention == "backward_anchored":
            out.append(t0 @ rel[i])
        else:
            raise ValueError(f"pose_convention must be one of {POSE_CONVENTIONS}")
    return np.stack(out)

"""Camera-pose helpers for render paths (reference role: the nerfstudio-derived helpers in
landmark/nerf_components/data/cameras.py:110-701): quaternion conversion and slerp, interpolation between key
poses (with intrinsics), smooth fly-through splines through many key poses, look-at construction, and
orientation / centring of a set of poses.  Poses are ``[3, 4]`` or ``[4, 4]`` camera-to-world matrices."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


def quaternion_from_matrix(R: np.ndarray) -> np.ndarray:
    """``(w, x, y, z)`` of a rotation matrix (Shepperd's method, w >= 0)."""
    R = np.asarray(R, dtype=np.float64)[:3, :3]
    t = np.trace(R)
    if t > 0:
        s = math.sqrt(t + 1.0) * 2
        q = np.array([0.25 * s, (R[2, 1] - R[1, 2]) / s, (R[0, 2] - R[2, 0]) / s, (R[1, 0] - R[0, 1]) / s])
    else:
        i = int(np.argmax(np.diag(R)))
        j, k = (i + 1) % 3, (i + 2) % 3
        s = math.sqrt(R[i, i] - R[j, j] - R[k, k] + 1.0) * 2
        q = np.zeros(4)
        q[0] = (R[k, j] - R[j, k]) / s
        q[1 + i] = 0.25 * s
        q[1 + j] = (R[j, i] + R[i, j]) / s
        q[1 + k] = (R[k, i] + R[i, k]) / s
    return q if q[0] >= 0 else -q


def quaternion_matrix(q: np.ndarray) -> np.ndarray:
    w, x, y, z = np.asarray(q, dtype=np.float64) / np.linalg.norm(q)
    return np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)],
                     [2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)],
                     [2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)]])


def quaternion_slerp(q0: np.ndarray, q1: np.ndarray, t: float) -> np.ndarray:
    q0, q1 = q0 / np.linalg.norm(q0), q1 / np.linalg.norm(q1)
    d = float(np.dot(q0, q1))
    if d < 0:
        q1, d = -q1, -d
    if d > 0.9995:
        q = q0 + t * (q1 - q0)
        return q / np.linalg.norm(q)
    theta = math.acos(d)
    return (math.sin((1 - t) * theta) * q0 + math.sin(t * theta) * q1) / math.sin(theta)


def get_interpolated_poses(pose_a: np.ndarray, pose_b: np.ndarray, steps: int = 10) -> List[np.ndarray]:
    """``steps`` poses from ``pose_a`` to ``pose_b`` inclusive: rotation by slerp, position linearly."""
    qa, qb = quaternion_from_matrix(pose_a[:3, :3]), quaternion_from_matrix(pose_b[:3, :3])
    out = []
    for t in np.linspace(0, 1, steps):
        pose = np.eye(4)
        pose[:3, :3] = quaternion_matrix(quaternion_slerp(qa, qb, float(t)))
        pose[:3, 3] = (1 - t) * pose_a[:3, 3] + t * pose_b[:3, 3]
        out.append(pose[:3])
    return out


def get_interpolated_k(k_a: np.ndarray, k_b: np.ndarray, steps: int = 10) -> List[np.ndarray]:
    return [(1 - t) * k_a + t * k_b for t in np.linspace(0, 1, steps)]


def get_interpolated_poses_many(poses: Sequence[np.ndarray], Ks: Optional[Sequence[np.ndarray]] = None,
                                steps_per_transition: int = 10) -> Tuple[np.ndarray, Optional[np.ndarray]]:
    """Piecewise interpolation through all key poses (and intrinsics); returns stacked ``[N, 3, 4]`` (and ``[N, 3, 3]``)."""
    traj, traj_k = [], []
    for i in range(len(poses) - 1):
        traj += get_interpolated_poses(np.asarray(poses[i]), np.asarray(poses[i + 1]), steps_per_transition)
        if Ks is not None:
            traj_k += get_interpolated_k(np.asarray(Ks[i]), np.asarray(Ks[i + 1]), steps_per_transition)
    return np.stack(traj), (np.stack(traj_k) if Ks is not None else None)


def catmull_rom_path(key_poses: Sequence[np.ndarray], n_frames: int) -> np.ndarray:
    """Smooth fly-through of ``n_frames`` poses through the key poses: positions on a centripetal-free uniform
    Catmull-Rom spline, rotations by slerp between the neighbouring keys."""
    keys = [np.asarray(p, dtype=np.float64) for p in key_poses]
    pos = np.array([k[:3, 3] for k in keys])
    quats = [quaternion_from_matrix(k[:3, :3]) for k in keys]
    n_seg = len(keys) - 1
    out = np.zeros((n_frames, 3, 4))
    for f in range(n_frames):
        u = f / max(n_frames - 1, 1) * n_seg
        i = min(int(u), n_seg - 1)
        t = u - i
        p0, p1, p2, p3 = pos[max(i - 1, 0)], pos[i], pos[i + 1], pos[min(i + 2, n_seg)]
        out[f, :, 3] = 0.5 * ((2 * p1) + (-p0 + p2) * t + (2 * p0 - 5 * p1 + 4 * p2 - p3) * t * t
                              + (-p0 + 3 * p1 - 3 * p2 + p3) * t ** 3)
        out[f, :, :3] = quaternion_matrix(quaternion_slerp(quats[i], quats[i + 1], t))
    return out


def normalize(v: np.ndarray) -> np.ndarray:
    return v / max(float(np.linalg.norm(v)), 1e-12)


def viewmatrix(lookat: np.ndarray, up: np.ndarray, pos: np.ndarray) -> np.ndarray:
    """Camera-to-world ``[3, 4]`` of a camera at ``pos`` looking along ``lookat`` (OpenGL axes: -z forward, y up)."""
    z = normalize(-np.asarray(lookat, dtype=np.float64))
    x = normalize(np.cross(np.asarray(up, dtype=np.float64), z))
    y = np.cross(z, x)
    return np.stack((x, y, z, np.asarray(pos, dtype=np.float64)), axis=1)


def focus_of_attention(poses: np.ndarray, initial_focus: np.ndarray) -> np.ndarray:
    """Point closest (least squares) to the optical axes of the cameras that look towards ``initial_focus``."""
    poses = np.asarray(poses, dtype=np.float64)
    origins, dirs = poses[:, :3, 3], -poses[:, :3, 2]
    active = np.einsum("ij,ij->i", dirs, initial_focus[None] - origins) > 0
    if not active.any():
        return initial_focus
    o, d = origins[active], dirs[active]
    m = np.eye(3)[None] - d[:, :, None] * d[:, None, :]
    return np.linalg.solve(m.sum(0), (m @ o[:, :, None]).sum(0)[:, 0])


def auto_orient_and_center_poses(poses: np.ndarray, method: str = "up", center_method: str = "poses"):
    """Rotate (``"up"``: mean camera up -> +z; ``"pca"``: principal axes; ``"none"``) and translate (``"poses"``: mean
    position; ``"focus"``: focus of attention; ``"none"``) a set of poses.  Returns ``(new_poses [N,3,4], transform [3,4])``."""
    poses = np.asarray(poses, dtype=np.float64)
    origins = poses[:, :3, 3]
    if center_method == "poses":
        t = origins.mean(0)
    elif center_method == "focus":
        t = focus_of_attention(poses, origins.mean(0))
    else:
        t = np.zeros(3)
    if method == "pca":
        centred = origins - t
        _, vecs = np.linalg.eigh(centred.T @ centred)
        R = vecs[:, ::-1].T
        if np.linalg.det(R) < 0:
            R[2] *= -1
        if (R @ poses[:, :3, 1].mean(0))[2] < 0:                      # keep the cameras' up direction pointing to +z
            R[1:] *= -1
    elif method == "up":
        up = normalize(poses[:, :3, 1].mean(0))
        z = np.array([0.0, 0.0, 1.0])
        v, c = np.cross(up, z), float(np.dot(up, z))
        if np.linalg.norm(v) < 1e-8:
            R = np.eye(3) if c > 0 else np.diag([1.0, -1.0, -1.0])
        else:
            vx = np.array([[0, -v[2], v[1]], [v[2], 0, -v[0]], [-v[1], v[0], 0]])
            R = np.eye(3) + vx + vx @ vx / (1 + c)
    else:
        R = np.eye(3)
    transform = np.concatenate((R, (R @ -t)[:, None]), axis=1)
    new = np.concatenate((R[None] @ poses[:, :3, :3], (R[None] @ (origins - t)[:, :, None])), axis=2)
    return new, transform


def poses_to_tensor(poses: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.as_tensor(np.asarray(poses), dtype=torch.float32, device=device)

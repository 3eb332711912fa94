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
                                steps_per_transition: int = 10, order_poses: bool = False
                                ) -> Tuple[np.ndarray, Optional[np.ndarray]]:
    """Piecewise interpolation through all key poses (and intrinsics); returns stacked ``[N, 3, 4]`` (and ``[N, 3, 3]``).
    ``order_poses`` first arranges the key poses as a greedy nearest-neighbour tour (:func:`get_ordered_poses_and_k`)."""
    if order_poses:
        stacked = torch.as_tensor(np.stack([np.asarray(p) for p in poses]), dtype=torch.float64)
        ks = torch.as_tensor(np.stack([np.asarray(k) for k in Ks]), dtype=torch.float64) if Ks is not None else \
            torch.zeros(len(poses), 3, 3, dtype=torch.float64)
        stacked, ks = get_ordered_poses_and_k(stacked, ks)
        poses, Ks = list(stacked.numpy()), (list(ks.numpy()) if Ks is not None else None)
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


# -- small vector / ordering / lens helpers (reference: landmark/nerf_components/data/cameras.py:111-127, 287-321,
# 364-376, 398-553) ------------------------------------------------------------------------------------------------
def unit_vector(data, axis: Optional[int] = None) -> np.ndarray:
    """``data`` scaled to unit Euclidean length along ``axis`` (the whole array when it is one-dimensional)."""
    v = np.array(data, dtype=np.float64)
    if v.ndim == 1 or axis is None:
        return v / np.sqrt(np.sum(v * v))
    return v / np.sqrt(np.sum(v * v, axis=axis, keepdims=True))


def normalize_with_norm(x: torch.Tensor, dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(x / |x|, |x|)`` along ``dim`` with the norm clamped away from zero."""
    norm = torch.linalg.vector_norm(x, dim=dim, keepdim=True).clamp_min(float(np.finfo(float).eps) * 4.0)
    return x / norm, norm


def get_ordered_poses_and_k(poses: torch.Tensor, Ks: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Greedy tour through the cameras: start at the first pose and always move to the nearest camera centre not yet
    visited.  ``poses [N, 3|4, 4]``, ``Ks [N, 3, 3]``; returns both in tour order."""
    n = poses.shape[0]
    centres = poses[:, :3, 3]
    left = torch.ones(n, dtype=torch.bool)
    order = [0]
    left[0] = False
    for _ in range(n - 1):
        d = torch.linalg.vector_norm(centres - centres[order[-1]], dim=1)
        d = torch.where(left, d, torch.full_like(d, float("inf")))
        nxt = int(torch.argmin(d))
        order.append(nxt)
        left[nxt] = False
    idx = torch.tensor(order, dtype=torch.long)
    return poses[idx], Ks[idx]


def get_distortion_params(k1: float = 0.0, k2: float = 0.0, k3: float = 0.0, k4: float = 0.0, p1: float = 0.0,
                          p2: float = 0.0) -> torch.Tensor:
    """OpenCV-style lens parameters as one vector ``[k1, k2, k3, k4, p1, p2]``."""
    return torch.tensor([k1, k2, k3, k4, p1, p2], dtype=torch.float32)


def radial_and_tangential_distort(coords: torch.Tensor, distortion_params: torch.Tensor) -> torch.Tensor:
    """Forward lens model on normalised image coordinates ``[..., 2]``: radial polynomial ``1 + k1 r^2 + k2 r^4 +
    k3 r^6 + k4 r^8`` and the two tangential terms."""
    k1, k2, k3, k4, p1, p2 = (distortion_params[..., i] for i in range(6))
    x, y = coords[..., 0], coords[..., 1]
    r2 = x * x + y * y
    radial = 1.0 + r2 * (k1 + r2 * (k2 + r2 * (k3 + r2 * k4)))
    xd = x * radial + 2.0 * p1 * x * y + p2 * (r2 + 2.0 * x * x)
    yd = y * radial + 2.0 * p2 * x * y + p1 * (r2 + 2.0 * y * y)
    return torch.stack((xd, yd), dim=-1)


def radial_and_tangential_undistort(coords: torch.Tensor, distortion_params: torch.Tensor, eps: float = 1e-3,
                                    max_iterations: int = 10) -> torch.Tensor:
    """Invert :func:`radial_and_tangential_distort` by Newton's method started at the distorted point; a point whose
    Jacobian determinant falls under ``eps`` stops moving."""
    k1, k2, k3, k4, p1, p2 = (distortion_params[..., i] for i in range(6))
    xd, yd = coords[..., 0], coords[..., 1]
    x, y = xd.clone(), yd.clone()
    for _ in range(max_iterations):
        r2 = x * x + y * y
        radial = 1.0 + r2 * (k1 + r2 * (k2 + r2 * (k3 + r2 * k4)))
        d_radial = k1 + r2 * (2.0 * k2 + r2 * (3.0 * k3 + r2 * 4.0 * k4))        # d radial / d r^2
        fx = x * radial + 2.0 * p1 * x * y + p2 * (r2 + 2.0 * x * x) - xd
        fy = y * radial + 2.0 * p2 * x * y + p1 * (r2 + 2.0 * y * y) - yd
        fx_x = radial + 2.0 * x * x * d_radial + 2.0 * p1 * y + 6.0 * p2 * x
        fx_y = 2.0 * x * y * d_radial + 2.0 * p1 * x + 2.0 * p2 * y
        fy_x = 2.0 * x * y * d_radial + 2.0 * p2 * y + 2.0 * p1 * x
        fy_y = radial + 2.0 * y * y * d_radial + 2.0 * p2 * x + 6.0 * p1 * y
        det = fx_x * fy_y - fx_y * fy_x
        ok = det.abs() > eps
        safe = torch.where(ok, det, torch.ones_like(det))
        x = x - torch.where(ok, (fx * fy_y - fy * fx_y) / safe, torch.zeros_like(det))
        y = y - torch.where(ok, (fy * fx_x - fx * fy_x) / safe, torch.zeros_like(det))
    return torch.stack((x, y), dim=-1)


def rotation_matrix(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """The rotation ``[3, 3]`` about ``a x b`` that turns the direction of ``a`` into the direction of ``b``
    (Rodrigues' formula); opposite vectors turn by pi about an axis perpendicular to ``a``."""
    a = a / torch.linalg.vector_norm(a)
    b = b / torch.linalg.vector_norm(b)
    v = torch.linalg.cross(a, b)
    c = torch.dot(a, b)
    if float(c) < -1.0 + 1e-8:
        helper = torch.eye(3, dtype=a.dtype)[int(torch.argmin(a.abs()))]
        axis = torch.linalg.cross(a, helper)
        axis = axis / torch.linalg.vector_norm(axis)
        return 2.0 * torch.outer(axis, axis) - torch.eye(3, dtype=a.dtype)
    K = torch.zeros(3, 3, dtype=a.dtype)
    K[0, 1], K[0, 2], K[1, 0], K[1, 2], K[2, 0], K[2, 1] = -v[2], v[1], v[2], -v[0], -v[1], v[0]
    return torch.eye(3, dtype=a.dtype) + K + K @ K / (1.0 + c)

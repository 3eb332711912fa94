"""Camera matrices in the row-vector convention used by the Gaussian models (reference:
landmark/nerf_components/utils/graphics_utils.py:19-123)."""
import math
from typing import NamedTuple

import numpy as np
import torch


class BasicPointCloud(NamedTuple):
    points: np.ndarray
    colors: np.ndarray
    normals: np.ndarray


def geom_transform_points(points, transf_matrix):
    ones = torch.ones(points.shape[0], 1, dtype=points.dtype, device=points.device)
    out = torch.cat((points, ones), dim=1) @ transf_matrix
    return out[:, :3] / (out[:, 3:4] + 1e-7)


def getWorld2View(R, t):
    Rt = np.zeros((4, 4), dtype=np.float32)
    Rt[:3, :3] = R.transpose()
    Rt[:3, 3] = t
    Rt[3, 3] = 1.0
    return Rt


def getWorld2View2(R, t, translate=np.array([0.0, 0.0, 0.0]), scale=1.0):
    """World->view with the camera centre re-expressed as ``(c + translate) * scale``."""
    Rt = getWorld2View(R, t)
    C2W = np.linalg.inv(Rt)
    C2W[:3, 3] = (C2W[:3, 3] + translate) * scale
    return np.linalg.inv(C2W).astype(np.float32)


def getProjectionMatrix(znear, zfar, fovX, fovY):
    tx, ty = math.tan(fovX / 2), math.tan(fovY / 2)
    top, right = ty * znear, tx * znear
    P = torch.zeros(4, 4)
    P[0, 0] = 2.0 * znear / (2 * right)
    P[1, 1] = 2.0 * znear / (2 * top)
    P[3, 2] = 1.0
    P[2, 2] = zfar / (zfar - znear)
    P[2, 3] = -(zfar * znear) / (zfar - znear)
    return P


def fov2focal(fov, pixels):
    return pixels / (2 * math.tan(fov / 2))


def focal2fov(focal, pixels):
    return 2 * math.atan(pixels / (2 * focal))


def pose_rotate_translate(c2w, rotation_deg=None, translation=None, *reference_tail, **reference_kw):
    """Apply a global Euler XYZ rotation (degrees) and translation to a camera-to-world matrix:
    ``pose_rotate_translate(c2w, [rx, ry, rz], [tx, ty, tz]) -> c2w'`` with ``c2w' = [R | t] c2w``.

    The reference's calling convention is accepted as well (graphics_utils.py:88-123):
    ``pose_rotate_translate(world_to_view, rot_x, rot_y, rot_z, trans) -> world_to_view'`` - the same motion applied to
    the inverse of the given matrix, result inverted back."""
    if reference_tail or reference_kw or not hasattr(rotation_deg, "__len__"):
        names = ("rot_x", "rot_y", "rot_z", "trans")
        positional = [v for v in (rotation_deg, translation) + tuple(reference_tail) if v is not None]
        given = dict(zip(names, positional))
        given.update(reference_kw)
        moved = pose_rotate_translate(np.linalg.inv(np.asarray(c2w, dtype=np.float64)),
                                      [given["rot_x"], given["rot_y"], given["rot_z"]], given["trans"])
        return np.linalg.inv(moved.astype(np.float64)).astype(np.float32)
    rx, ry, rz = [math.radians(float(a)) for a in rotation_deg]
    Rx = np.array([[1, 0, 0], [0, math.cos(rx), -math.sin(rx)], [0, math.sin(rx), math.cos(rx)]])
    Ry = np.array([[math.cos(ry), 0, math.sin(ry)], [0, 1, 0], [-math.sin(ry), 0, math.cos(ry)]])
    Rz = np.array([[math.cos(rz), -math.sin(rz), 0], [math.sin(rz), math.cos(rz), 0], [0, 0, 1]])
    M = np.eye(4)
    M[:3, :3] = Rz @ Ry @ Rx
    M[:3, 3] = np.asarray(translation, dtype=np.float64)
    return (M @ np.asarray(c2w, dtype=np.float64)).astype(np.float32)

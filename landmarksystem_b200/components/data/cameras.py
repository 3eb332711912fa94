"""Pinhole camera record used by the Gaussian-splatting models (reference:
landmark/nerf_components/data/cameras.py:34-108).  Matrices follow the row-vector convention:
``world_view_transform`` is the transposed world-to-view matrix, ``full_proj_transform = W @ P``."""
from __future__ import annotations

import math
from dataclasses import dataclass, field, fields
from typing import Optional

import numpy as np
import torch

from ..utils.graphics_utils import getProjectionMatrix, getWorld2View2


@dataclass
class Camera:
    uid: int = 0
    image_width: int = 0
    image_height: int = 0
    FoVx: float = 0.0
    FoVy: float = 0.0
    R: Optional[np.ndarray] = None          # camera-to-world rotation (COLMAP axes)
    T: Optional[np.ndarray] = None          # world-to-camera translation
    znear: float = 0.01
    zfar: float = 100.0
    trans: np.ndarray = field(default_factory=lambda: np.zeros(3))
    scale: float = 1.0
    image: Optional[torch.Tensor] = None
    image_name: str = ""
    image_path: str = ""
    resolution_scale: float = 1.0
    world_view_transform: Optional[torch.Tensor] = None
    projection_matrix: Optional[torch.Tensor] = None
    full_proj_transform: Optional[torch.Tensor] = None
    camera_center: Optional[torch.Tensor] = None

    def __post_init__(self):
        if self.world_view_transform is None and self.R is not None:
            w2v = torch.tensor(getWorld2View2(self.R, self.T, self.trans, self.scale)).transpose(0, 1)
            proj = getProjectionMatrix(self.znear, self.zfar, self.FoVx, self.FoVy).transpose(0, 1)
            self.world_view_transform = w2v
            self.projection_matrix = proj
            self.full_proj_transform = w2v @ proj
            self.camera_center = w2v.inverse()[3, :3]

    # -- the reference's field names (landmark/nerf_components/data/cameras.py:33-66) as read-only views --------
    @property
    def width(self) -> int:
        return self.image_width

    @property
    def height(self) -> int:
        return self.image_height

    @property
    def FovX(self) -> float:
        return self.FoVx

    @property
    def FovY(self) -> float:
        return self.FoVy

    @property
    def device(self):
        return self.world_view_transform.device if self.world_view_transform is not None else torch.device("cpu")

    @property
    def c2w(self) -> Optional[torch.Tensor]:
        """Camera-to-world matrix ``[4, 4]`` in COLMAP axes (x right, y down, z forward).  Assignable: adapters of the
        reference clear it (``cam.c2w = None``) before a camera travels to other ranks."""
        if "_c2w" in self.__dict__:
            return self.__dict__["_c2w"]
        if self.world_view_transform is None:
            return None
        return torch.linalg.inv(self.world_view_transform.transpose(0, 1))

    @c2w.setter
    def c2w(self, value) -> None:
        self.__dict__["_c2w"] = value

    @property
    def tanfovx(self) -> float:
        return math.tan(self.FoVx * 0.5)

    @property
    def tanfovy(self) -> float:
        return math.tan(self.FoVy * 0.5)

    def to(self, device, non_blocking: bool = False) -> "Camera":
        moved = {}
        for f in fields(self):
            value = getattr(self, f.name)
            moved[f.name] = value.to(device, non_blocking=non_blocking) if torch.is_tensor(value) else value
        cam = object.__new__(Camera)
        cam.__dict__.update(moved)
        return cam

    def cuda(self):
        return self.to("cuda")

    def cpu(self):
        return self.to("cpu")

    @staticmethod
    def from_c2w(c2w_opengl: np.ndarray, width: int, height: int, focal_x: float, focal_y: Optional[float] = None,
                 uid: int = 0, image=None, znear: float = 0.01, zfar: float = 100.0, image_name: str = "") -> "Camera":
        """Build from an OpenGL-convention camera-to-world matrix (the transforms.json convention)."""
        c2w = np.array(c2w_opengl, dtype=np.float64).copy()
        c2w[:3, 1:3] *= -1.0                      # OpenGL (y up, -z fwd) -> COLMAP (y down, +z fwd)
        w2c = np.linalg.inv(c2w)
        R = np.transpose(w2c[:3, :3])
        T = w2c[:3, 3]
        focal_y = focal_y or focal_x
        fovx = 2 * math.atan(width / (2 * focal_x))
        fovy = 2 * math.atan(height / (2 * focal_y))
        return Camera(uid=uid, image_width=width, image_height=height, FoVx=fovx, FoVy=fovy,
                      R=R.astype(np.float32), T=T.astype(np.float32), znear=znear, zfar=zfar, image=image,
                      image_name=image_name)

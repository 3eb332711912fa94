"""3DGS-family datasets on COLMAP reconstructions.

``ColmapGaussianDataset`` (reference role: .../dataloader/colmap_dataset.py:25-176): ``<datadir>/sparse/0`` +
``<datadir>/images[_k]``; every ``llffhold``-th image (sorted by name) is the test split when ``eval`` is set;
camera centres are shifted/scaled so that training cameras fit a unit-ish sphere (``nerf_normalization``);
the sparse point cloud is exposed for initialisation.

``ZhangjiangGaussianDataset`` (reference role: .../dataloader/zhangjiang_dataset.py): the same layout for the
aerial survey scene, with a metric world whose origin is moved to the centroid of the cameras and an optional
axis-aligned crop (``lb`` / ``ub``) applied to both cameras and points."""
from __future__ import annotations

import math
import os
from typing import List

import numpy as np

from ..cameras import Camera
from .base_dataset import GaussianSplattingDataset
from .colmap_loader import read_model


def _fov(focal: float, pixels: int) -> float:
    return 2.0 * math.atan(pixels / (2.0 * focal))


def nerf_normalization(centers: np.ndarray):
    """``(translate, radius)``: centre of the camera positions and 1.1 x the largest distance to it."""
    mean = centers.mean(axis=0)
    radius = float(np.linalg.norm(centers - mean, axis=1).max()) * 1.1 if len(centers) else 1.0
    return -mean, radius


class ColmapGaussianDataset(GaussianSplattingDataset):
    llffhold = 8

    def __init__(self, split="train", downsample=1.0, args=None, preload=False):
        super().__init__(split, downsample, args, preload)
        self._build(args, split, float(downsample), preload, recentre=False, crop=False)

    # shared with the subclass
    def _build(self, args, split, ds, preload, recentre: bool, crop: bool):
        sparse = os.path.join(args.datadir, "sparse", "0")
        if not os.path.isdir(sparse):
            sparse = os.path.join(args.datadir, "sparse")
        cams, images, (xyz, rgb, _) = read_model(sparse)
        image_dir = getattr(args, "images", None) or "images"
        if ds > 1 and os.path.isdir(os.path.join(args.datadir, f"{image_dir}_{int(ds)}")):
            image_dir = f"{image_dir}_{int(ds)}"
        ordered = sorted(images.values(), key=lambda im: im.name)
        centres = np.array([-(im.rotation().T @ im.tvec) for im in ordered]).reshape(-1, 3)
        shift = -centres.mean(axis=0) if (recentre and len(centres)) else np.zeros(3)
        lb = np.array(getattr(args, "lb", None) or [-np.inf] * 3, dtype=np.float64)
        ub = np.array(getattr(args, "ub", None) or [np.inf] * 3, dtype=np.float64)
        hold = bool(getattr(args, "eval", True))
        cameras: List[Camera] = []
        for k, im in enumerate(ordered):
            is_test = hold and (k % self.llffhold == 0)
            if (split == "train" and is_test) or (split != "train" and hold and not is_test):
                continue
            centre = centres[k] + shift
            if crop and (np.any(centre[:2] < lb[:2]) or np.any(centre[:2] > ub[:2])):
                continue
            cc = cams[im.camera_id]
            fx, fy = cc.focal()
            ds_cam = ds * self.resolution_factor(cc.width)
            W, H = int(round(cc.width / ds_cam)), int(round(cc.height / ds_cam))
            R = im.rotation().T                                   # camera-to-world rotation, as Camera.R expects
            T = im.tvec - im.rotation() @ shift                   # world moved by `shift`
            cam = Camera(uid=len(cameras), image_width=W, image_height=H, FoVx=_fov(fx / ds_cam, W), FoVy=_fov(fy / ds_cam, H),
                         R=R.astype(np.float32), T=T.astype(np.float32), image_name=os.path.basename(im.name))
            cam.image_path = os.path.join(args.datadir, image_dir, im.name)
            if preload:
                cam.image = self.load_image(cam)
            cameras.append(cam)
        self.cameras = cameras
        pts = xyz + shift
        if crop and len(pts):
            keep = np.all(pts >= lb, axis=1) & np.all(pts <= ub, axis=1)
            pts, rgb = pts[keep], rgb[keep]
        self.points_xyz, self.points_rgb = pts.astype(np.float32), (rgb.astype(np.float32) / 255.0)
        self.translate, self.radius = nerf_normalization(np.array([c.camera_center.numpy() for c in cameras]).reshape(-1, 3))
        self.cameras_extent = self.radius
        self.world_shift = shift
        self.white_bg = bool(getattr(args, "white_bkgd", False))

    def initial_point_cloud(self):
        """``(xyz [N,3], rgb [N,3] in [0,1])`` of the sparse reconstruction (initial Gaussians / anchors)."""
        return self.points_xyz, self.points_rgb


class ZhangjiangGaussianDataset(ColmapGaussianDataset):
    llffhold = 10

    def __init__(self, split="train", downsample=1.0, args=None, preload=False):
        GaussianSplattingDataset.__init__(self, split, downsample, args, preload)
        self._build(args, split, float(downsample), preload, recentre=True, crop=True)

"""transforms.json-based datasets: MatrixCity, City (+ Gaussian variant) and Blender (reference:
.../dataloader/matrixcity_dataset.py:17-515, city_dataset.py:27-654, blender_dataset.py:29-132).

All three read ``datadir/transforms_{split}.json`` with OpenGL camera-to-world matrices; they differ
in where images live and how the focal length is given.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional

import numpy as np
import torch

from ..cameras import Camera
from .base_dataset import GaussianSplattingDataset, VolumeRenderDataset
from .ray_utils import frames_to_poses, load_transforms


def _read_image(path: str, W: int, H: int, white_bg: bool) -> torch.Tensor:
    from PIL import Image

    img = Image.open(path)
    if (img.width, img.height) != (W, H):
        img = img.resize((W, H), Image.LANCZOS)
    arr = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0)
    if arr.dim() == 2:
        arr = arr[..., None].expand(-1, -1, 3)
    if arr.shape[-1] == 4:
        rgb, a = arr[..., :3], arr[..., 3:4]
        arr = rgb * a + (1.0 - a) if white_bg else rgb * a
    return arr[..., :3].reshape(-1, 3).contiguous()


def _resolve(datadir: str, file_path: str, sub: Optional[str] = None) -> str:
    cands = [os.path.join(datadir, file_path)]
    if sub:
        cands.append(os.path.join(datadir, sub, os.path.basename(file_path)))
    for c in list(cands):
        cands += [c + ".png", c + ".jpg"]
    for c in cands:
        if os.path.isfile(c):
            return c
    return cands[0]


class _JsonNeRFDataset(VolumeRenderDataset):
    image_subdir: Optional[str] = None

    def __init__(self, split="train", downsample=1.0, is_stack=False, args=None, enable_lpips=False,
                 load_images=True):
        super().__init__(split, downsample, is_stack, args)
        self.datadir = args.datadir
        self.near_far = list(getattr(args, "train_near_far", None) or [0.1, 10.0])
        self.white_bg = bool(getattr(args, "white_bkgd", False))
        self.enable_lpips = enable_lpips
        if split == "path":                          # fly-around or trajectory file: poses only, no images
            self.read_meta_path()
            return
        meta = load_transforms(self.datadir, split)
        W, H, focal = self.intrinsics(meta)
        paths, poses = frames_to_poses(meta)
        poses = self.transform_poses(poses)
        self.image_paths = [_resolve(self.datadir, p, self.image_subdir) for p in paths]
        images = [_read_image(p, W, H, self.white_bg) for p in self.image_paths] if load_images else None
        self.build_rays(torch.from_numpy(poses), images, H, W, focal, getattr(args, "camera", "normal"))

    def intrinsics(self, meta):
        ds = float(self.downsample)
        W, H = int(meta.get("w", 1920) / ds), int(meta.get("h", 1080) / ds)
        return W, H, float(meta["fl_x"]) / ds

    def transform_poses(self, poses: np.ndarray) -> np.ndarray:
        return poses


class MatrixCityDataset(_JsonNeRFDataset):
    """Images are addressed relative to ``datadir``; focal = ``fl_x / downsample``."""


class CityDataset(_JsonNeRFDataset):
    """Images live in ``images_{downsample}/``; a global pose rotation/translation may be applied."""

    def __init__(self, *a, **kw):
        args = kw.get("args") or a[3]
        self.image_subdir = f"images_{int(kw.get('downsample', 1) or 1)}"
        self._rot = getattr(args, "pose_rotation", [0, 0, 0])
        self._trans = getattr(args, "pose_translation", [0, 0, 0])
        super().__init__(*a, **kw)

    def transform_poses(self, poses):
        from ...utils.graphics_utils import pose_rotate_translate

        if any(float(v) != 0 for v in list(self._rot) + list(self._trans)):
            return np.stack([pose_rotate_translate(p, self._rot, self._trans) for p in poses])
        return poses


class BlenderDataset(_JsonNeRFDataset):
    """NeRF-synthetic: ``camera_angle_x`` gives the focal length; 800x800 RGBA images, white bg."""

    def intrinsics(self, meta):
        ds = float(self.downsample)
        W = H = int(800 / ds)
        return W, H, 0.5 * W / math.tan(0.5 * float(meta["camera_angle_x"]))


class CityGaussianDataset(GaussianSplattingDataset):
    """Camera list for the 3DGS family from the same transforms.json files (reference:
    city_dataset.py:568-654): c2w flipped to COLMAP axes, znear 0.01 / zfar 100."""

    def __init__(self, split="train", downsample=1.0, args=None, preload=False):
        super().__init__(split, downsample, args, preload)
        from ...utils.graphics_utils import pose_rotate_translate

        meta = load_transforms(args.datadir, split)
        ds = float(downsample)
        W, H = int(meta.get("w", 1920) / ds), int(meta.get("h", 1080) / ds)
        fx = float(meta["fl_x"]) / ds
        fy = float(meta.get("fl_y", meta["fl_x"])) / ds
        paths, poses = frames_to_poses(meta)
        rot, trans = getattr(args, "pose_rotation", [0, 0, 0]), getattr(args, "pose_translation", [0, 0, 0])
        for k, (p, c2w) in enumerate(zip(paths, poses)):
            if any(float(v) != 0 for v in list(rot) + list(trans)):
                c2w = pose_rotate_translate(c2w, rot, trans)
            cam = Camera.from_c2w(c2w, W, H, fx, fy, uid=k, image_name=os.path.basename(p))
            cam.image_path = _resolve(args.datadir, p, f"images_{int(ds)}")
            if preload:
                cam.image = self.load_image(cam)
            self.cameras.append(cam)
        self.white_bg = bool(getattr(args, "white_bkgd", False))
        self.compute_extent()

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
        """``(W, H, focal)``; ``focal`` is one number, or an array with one focal length per frame when the file gives
        ``fl_x`` inside the frames (the reference's drone layout, ray_utils.py:122-170; one image size for all)."""
        ds = float(self.downsample)
        frames = meta.get("frames", [])
        first = frames[0] if frames else {}
        W = int(meta.get("w", first.get("w", 1920)) / ds)
        H = int(meta.get("h", first.get("h", 1080)) / ds)
        if "fl_x" in meta:
            return W, H, float(meta["fl_x"]) / ds
        if "fl_x" in first:
            return W, H, np.asarray([float(f["fl_x"]) for f in frames], dtype=np.float64) / ds
        assert "camera_angle_x" in meta, "transforms file gives neither a focal length nor camera_angle_x"
        return W, H, 0.5 * W / math.tan(0.5 * float(meta["camera_angle_x"]))

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
        paths, poses = frames_to_poses(meta)
        rot, trans = getattr(args, "pose_rotation", [0, 0, 0]), getattr(args, "pose_translation", [0, 0, 0])
        for k, (p, c2w, frame) in enumerate(zip(paths, poses, meta["frames"])):
            if any(float(v) != 0 for v in list(rot) + list(trans)):
                c2w = pose_rotate_translate(c2w, rot, trans)
            path = _resolve(args.datadir, p, f"images_{int(ds)}")
            W, H, fx, fy = self._intrinsics(meta, frame, path, ds)
            cam = Camera.from_c2w(c2w, W, H, fx, fy, uid=k, image_name=os.path.basename(p))
            cam.image_path = path
            if preload:
                cam.image = self.load_image(cam)
            self.cameras.append(cam)
        self.white_bg = bool(getattr(args, "white_bkgd", False))
        self.compute_extent()

    _size_cache = None

    def _intrinsics(self, meta, frame, image_path: str, ds: float):
        """``(W, H, fx, fy)`` of one frame.  Three layouts of ``transforms_*.json`` are read (reference:
        city_dataset.py:568-612 and the data-preparation page of its documentation): one focal length for the whole
        file (``fl_x`` [, ``fl_y``, ``w``, ``h``]), one field of view (``camera_angle_x``), or focal length and size per
        frame.  A size that the file does not give is taken from the image itself (read once when it is global)."""
        def size_of(scope):
            if "w" in scope and "h" in scope:
                return int(scope["w"]), int(scope["h"])
            return None

        size = size_of(frame) or size_of(meta)
        if size is None:
            if "fl_x" in frame or self._size_cache is None:
                if os.path.isfile(image_path):
                    from PIL import Image

                    with Image.open(image_path) as im:
                        size = im.size
                else:
                    size = (1920, 1080)                  # the MatrixCity frame size
                if "fl_x" not in frame:
                    self._size_cache = size
            else:
                size = self._size_cache
        W0, H0 = size
        if "fl_x" in frame:
            fx0, fy0 = float(frame["fl_x"]), float(frame.get("fl_y", frame["fl_x"]))
        elif "fl_x" in meta:
            fx0, fy0 = float(meta["fl_x"]), float(meta.get("fl_y", meta["fl_x"]))
        else:
            assert "camera_angle_x" in meta, "transforms file gives neither a focal length nor camera_angle_x"
            fx0 = fy0 = 0.5 * W0 / math.tan(0.5 * float(meta["camera_angle_x"]))
        ds = ds * self.resolution_factor(W0)
        return int(W0 / ds), int(H0 / ds), fx0 / ds, fy0 / ds

"""Dataset base classes (reference:
landmark/nerf_components/data/datasets/dataloader/base_dataset.py:23-358).

``VolumeRenderDataset`` precomputes every ray on the host: ``all_rays [N, 6]``, ``all_rgbs [N, 3]``,
``all_idxs [N]`` for training (flat) and ``[n_img, H*W, ...]`` for testing.
``GaussianSplattingDataset`` is a list of :class:`Camera` records with (lazily loaded) images.
"""
from __future__ import annotations

import os
from typing import List, Optional

import numpy as np
import torch
from torch.utils.data import Dataset

from ..cameras import Camera
from .ray_utils import get_ray_directions_blender, get_rays, load_json_render_path, pose_spherical


def _arg(args, name, default):
    """``args.name`` of a namespace / mapping-like configuration, ``default`` when absent or ``None``-less."""
    if args is None:
        return default
    value = args.get(name, default) if hasattr(args, "get") else getattr(args, name, default)
    return default if value is None else value


class _Overlay:
    """A configuration seen through a dictionary of overrides."""

    def __init__(self, base, over):
        self._base, self._over = base, over

    def get(self, name, default=None):
        if name in self._over:
            return self._over[name]
        return _arg(self._base, name, default)

    def __getattr__(self, name):
        value = self.get(name, None)
        if value is None:
            raise AttributeError(name)
        return value


class BaseDataset(Dataset):
    def __init__(self, split: str = "train", downsample: float = 1.0, is_stack: bool = False, args=None):
        self.split, self.downsample, self.is_stack, self.args = split, downsample, is_stack, args
        self.white_bg = False
        self.near_far = [0.1, 10.0]
        self.scene_bbox = None
        self.image_paths: List[str] = []


class VolumeRenderDataset(BaseDataset):
    def __init__(self, split="train", downsample=1.0, is_stack=False, args=None):
        super().__init__(split, downsample, is_stack, args)
        self.all_rays = self.all_rgbs = self.all_idxs = None
        self.img_wh = (0, 0)
        self.focal = None
        self.poses = None
        if args is not None:
            self.scene_bbox = torch.tensor([list(args.lb), list(args.ub)], dtype=torch.float32)

    def build_rays(self, poses: torch.Tensor, images: Optional[List[torch.Tensor]], H: int, W: int, focal,
                   camera_mode: str = "normal"):
        """Fill ``all_rays/all_rgbs/all_idxs`` from per-image poses (OpenGL c2w) and ``[H*W, 3]`` images.  ``focal``:
        one number (or an ``(fx, fy)`` tuple) for every image, or a one-dimensional numpy array with one focal length
        per image."""
        per_image = isinstance(focal, np.ndarray) and focal.ndim == 1
        assert not per_image or len(focal) == len(poses), "one focal length per image"
        dirs = None if per_image else get_ray_directions_blender(H, W, focal)
        rays, idxs = [], []
        for k, c2w in enumerate(poses):
            if per_image:
                dirs = get_ray_directions_blender(H, W, float(focal[k]))
            o, d = get_rays(dirs, torch.as_tensor(c2w, dtype=torch.float32), camera_mode)
            rays.append(torch.cat((o, d), -1))
            idxs.append(torch.full((H * W,), float(k)))
        self.img_wh, self.focal, self.poses = (W, H), focal, poses
        if self.is_stack:
            self.all_rays = torch.stack(rays)
            self.all_idxs = torch.stack(idxs)
            self.all_rgbs = torch.stack(images) if images is not None else None
        else:
            self.all_rays = torch.cat(rays)
            self.all_idxs = torch.cat(idxs)
            self.all_rgbs = torch.cat(images) if images is not None else None

    def render_path_poses(self) -> torch.Tensor:
        """Camera-to-world matrices ``[n, 4, 4]`` of the ``"path"`` split.

        ``render_spherical``: ``render_nframes // render_skip`` cameras on ``render_ncircle`` turns of a circle of
        radius ``render_spherical_radius`` looking ``render_downward`` degrees down, moved to ``self.cxyz`` when the
        dataset has a scene centre, descending by ``render_spherical_zdiff`` over the first half of the frames and
        climbing back over the second.  Otherwise the frames of ``datadir/trajectories/path{render_pathid}.json``
        (``{"frames": [{"transform_matrix": ...}]}``), every ``render_skip``-th.
        """
        a = self.args
        skip = max(int(_arg(a, "render_skip", 1)), 1)
        if bool(_arg(a, "render_spherical", False)):
            n = max(int(_arg(a, "render_nframes", 100)) // skip, 1)
            radius = float(_arg(a, "render_spherical_radius", 4.0))
            downward = float(_arg(a, "render_downward", -45.0))
            zdiff = float(_arg(a, "render_spherical_zdiff", 1.0))
            angles = np.linspace(0.0, 360.0 * float(_arg(a, "render_ncircle", 1)), n + 1)[:-1]
            poses = torch.stack([pose_spherical(float(t), downward, radius) for t in angles])
            centre = getattr(self, "cxyz", None)
            if centre is not None:
                poses[:, :3, 3] += torch.as_tensor(centre, dtype=torch.float32)[:3]
            if zdiff > 0:
                half, zstep = n // 2, zdiff / n * 2
                k = torch.arange(n, dtype=torch.float32)
                poses[:, 2, 3] -= torch.where(k < half, zstep * k, zdiff - zstep * (k - half))
            return poses
        poses = load_json_render_path(os.path.join(self.datadir, "trajectories"),
                                      f"path{int(_arg(a, 'render_pathid', 0))}.json", skip)
        return torch.as_tensor(poses, dtype=torch.float32)

    def read_meta_path(self, n_frames: Optional[int] = None, radius: Optional[float] = None,
                       downward: Optional[float] = None):
        """Rays of the ``"path"`` split: poses only, no images (reference: base_dataset.py:151-214).

        The image is ``render_px`` rows of 16:9 with the focal length of ``render_fov`` degrees (over the rows); near /
        far planes and the bounding box come from ``render_near_far`` / ``render_lb`` / ``render_ub`` when set.  The
        keyword arguments override the configured spherical path (frame count, radius, downward angle).
        """
        a = self.args
        if n_frames is not None or radius is not None or downward is not None:
            over = {"render_spherical": True, "render_skip": 1, "render_spherical_zdiff": 0.0}
            if n_frames is not None:
                over["render_nframes"] = n_frames
            if radius is not None:
                over["render_spherical_radius"] = radius
            if downward is not None:
                over["render_downward"] = downward
            self.args = _Overlay(a, over)
        try:
            poses = self.render_path_poses()
        finally:
            self.args = a
        if a is not None and _arg(a, "render_px", None) and self.split == "path":
            H = int(_arg(a, "render_px", 720))
            W = int(1920 / 1080 * H)
            focal = 0.5 * H / np.tan(0.5 * np.deg2rad(float(_arg(a, "render_fov", 65.0))))
        else:
            (W, H), focal = self.img_wh, self.focal
        if a is not None and _arg(a, "render_near_far", None):
            self.near_far = list(a.render_near_far)
        if a is not None and _arg(a, "render_lb", None) and _arg(a, "render_ub", None):
            self.render_scene_bbox = torch.tensor([list(a.render_lb), list(a.render_ub)], dtype=torch.float32)
        self.is_stack = True
        self.build_rays(poses, None, H, W, focal, _arg(a, "camera", "normal"))
        self.render_poses, self.render_rays = poses, self.all_rays

    def preprocess(self, args=None, batch_size: int = 8192, root: Optional[str] = None) -> int:
        """Shuffle this dataset's rays and write them as shards of ``batch_size`` rays under ``root`` (default
        ``args.preprocessed_dir``); returns the number of shards (reference: matrixcity_dataset.py:113-302)."""
        from .processed_dataset import preprocess

        flat = self._flat_view()
        return preprocess(flat, root or (args or self.args).preprocessed_dir, shard_rays=batch_size)

    def distpreprocess(self, args=None, batch_size: int = 8192, root: Optional[str] = None, group=None) -> int:
        """The same collectively: every rank of the default group writes its share of the shards (reference:
        matrixcity_dataset.py:304-515)."""
        import torch.distributed as dist

        from .processed_dataset import dist_preprocess

        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        return dist_preprocess(self._flat_view(), root or (args or self.args).preprocessed_dir, rank, world,
                               shard_rays=batch_size, group=group)

    def _flat_view(self):
        from types import SimpleNamespace

        assert self.all_rgbs is not None, "this split has no colours to store"
        return SimpleNamespace(all_rays=self.all_rays.reshape(-1, self.all_rays.shape[-1]),
                               all_rgbs=self.all_rgbs.reshape(-1, 3), all_idxs=self.all_idxs.reshape(-1))

    def __len__(self):
        return 0 if self.all_rays is None else self.all_rays.shape[0]

    def __getitem__(self, i):
        item = {"rays": self.all_rays[i], "idxs": self.all_idxs[i]}
        if self.all_rgbs is not None:
            item["rgbs"] = self.all_rgbs[i]
        return item


class GaussianSplattingDataset(BaseDataset):
    def __init__(self, split="train", downsample=1.0, args=None, preload: bool = False):
        super().__init__(split, downsample, True, args)
        self.cameras: List[Camera] = []
        self.preload = preload
        self.cameras_extent = 1.0

    def resolution_factor(self, original_width: int, resolution_scale: float = 1.0) -> float:
        """Extra size divisor from the ``resolution`` field of the configuration (reference:
        base_dataset.py:344-358): ``-1`` keeps the size, ``1 / 2 / 4 / 8`` divide it, any other number is the target
        width in pixels; ``resolution_scale`` multiplies the divisor (multi-scale training).  Camera size, focal length
        and the loaded image all follow the same divisor, so renders and ground truth keep matching."""
        resolution = getattr(self.args, "resolution", -1) if self.args is not None else -1
        resolution = -1 if resolution is None else resolution
        if resolution == -1:
            return float(resolution_scale)
        if resolution in (1, 2, 4, 8):
            return float(resolution) * float(resolution_scale)
        return float(original_width) / float(resolution) * float(resolution_scale)

    def load_image(self, cam: Camera) -> torch.Tensor:
        if cam.image is not None:
            return cam.image
        from PIL import Image

        img = Image.open(cam.image_path).convert("RGB")
        if (img.width, img.height) != (cam.image_width, cam.image_height):
            img = img.resize((cam.image_width, cam.image_height), Image.LANCZOS)
        return torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1).contiguous()

    @property
    def resolution_scales(self) -> List[float]:
        scales = getattr(self.args, "resolution_scales", None) if self.args is not None else None
        return [float(s) for s in scales] if scales else [1.0]

    def __len__(self):
        return len(self.cameras) * len(self.resolution_scales)

    def __getitem__(self, i):
        """Item ``i`` is camera ``i // n_scales`` at scale ``i % n_scales`` of ``resolution_scales`` (reference:
        base_dataset.py:314-331): the same view with width and height divided by the scale (field of view unchanged),
        ``resolution_scale`` set on the camera - Octree-GS picks coarser levels for it - and the image loaded at that size."""
        scales = self.resolution_scales
        cam = self.cameras[i // len(scales)]
        scale = scales[i % len(scales)]
        if scale != 1.0:
            import dataclasses

            full = cam.image
            cam = dataclasses.replace(cam, image_width=max(int(round(cam.image_width / scale)), 1),
                                      image_height=max(int(round(cam.image_height / scale)), 1),
                                      resolution_scale=scale, image=None)
            if full is not None:                 # images held in memory (preloaded / synthetic): resample them
                cam.image = torch.nn.functional.interpolate(full[None].float(), size=(cam.image_height, cam.image_width),
                                                            mode="bilinear", align_corners=False, antialias=True)[0]
        return cam, self.load_image(cam)

    @staticmethod
    def collate_fn(batch):
        """One camera per step: return the first (camera, image) pair."""
        return batch[0]

    def compute_extent(self):
        """Radius of the camera cloud (``getNeRFppNorm``): 1.1 x max distance to the mean centre."""
        centers = torch.stack([c.camera_center for c in self.cameras])
        self.cameras_extent = float((centers - centers.mean(0)).norm(dim=-1).max() * 1.1)
        return self.cameras_extent

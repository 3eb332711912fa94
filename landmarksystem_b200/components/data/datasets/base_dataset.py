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
from .ray_utils import get_ray_directions_blender, get_rays, pose_spherical


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
        """Fill ``all_rays/all_rgbs/all_idxs`` from per-image poses (OpenGL c2w) and ``[H*W, 3]`` images."""
        dirs = get_ray_directions_blender(H, W, focal)
        rays, idxs = [], []
        for k, c2w in enumerate(poses):
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

    def read_meta_path(self, n_frames: int = 100, radius: float = 4.0, downward: float = -45.0):
        """Spherical render path (``render_spherical``): poses only, no images."""
        poses = torch.stack([pose_spherical(a, downward, radius) for a in np.linspace(-180, 180, n_frames + 1)[:-1]])
        W, H = self.img_wh
        self.is_stack = True
        self.build_rays(poses, None, H, W, self.focal)

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

    def load_image(self, cam: Camera) -> torch.Tensor:
        if cam.image is not None:
            return cam.image
        from PIL import Image

        img = Image.open(cam.image_path).convert("RGB")
        if (img.width, img.height) != (cam.image_width, cam.image_height):
            img = img.resize((cam.image_width, cam.image_height), Image.LANCZOS)
        return torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1).contiguous()

    def __len__(self):
        return len(self.cameras)

    def __getitem__(self, i):
        cam = self.cameras[i]
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

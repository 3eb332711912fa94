"""Procedural datasets (``dataset_name="synthetic"``): an analytic Gaussian-blob scene rendered from a
camera rig.  No files are read; ``datadir`` selects the rig: ``"ring:<n>:<HxW>:<focal>:<radius>"`` or
``"aerial:<n>:<HxW>:<focal>:<altitude>"`` (missing fields take defaults).  They replace the private
MatrixCity captures the reference's tests depend on."""
from __future__ import annotations

import math

import numpy as np
import torch

from ....synthetic.scene import BlobField, aerial_cameras, make_blob_dataset, ring_cameras
from ..cameras import Camera
from .base_dataset import GaussianSplattingDataset, VolumeRenderDataset


def _parse(datadir: str):
    parts = (datadir or "ring").split(":")
    kind = parts[0] if parts[0] in ("ring", "aerial") else "ring"
    n = int(parts[1]) if len(parts) > 1 and parts[1] else 8
    H, W = (int(v) for v in parts[2].split("x")) if len(parts) > 2 and parts[2] else (64, 64)
    focal = float(parts[3]) if len(parts) > 3 and parts[3] else 80.0
    extra = float(parts[4]) if len(parts) > 4 and parts[4] else (3.0 if kind == "ring" else 400.0)
    return kind, n, H, W, focal, extra


def _rig(args, split):
    kind, n, H, W, focal, extra = _parse(args.datadir)
    lb, ub = list(args.lb), list(args.ub)
    n_blobs = int(getattr(args, "synthetic_blobs", 32))
    field = BlobField.random(n_blobs, lb, ub, seed=int(getattr(args, "synthetic_seed", 0)))
    if kind == "ring":
        n_cam = n if split == "train" else max(n // 4, 1)
        poses = ring_cameras(n_cam, extra, height=0.0 if split == "train" else 0.3 * extra,
                             target=tuple((np.array(lb) + np.array(ub)) / 2))
        near, far = max(extra - 1.5 * float(np.linalg.norm(np.array(ub) - np.array(lb))) / 2, 0.05), \
            extra + 1.5 * float(np.linalg.norm(np.array(ub) - np.array(lb))) / 2
    else:
        poses = aerial_cameras(n if split == "train" else max(n // 4, 1), lb, ub, extra,
                               seed=0 if split == "train" else 1)
        near, far = 0.05 * extra, 2.0 * extra
    nf = getattr(args, "train_near_far", None)
    if nf:
        near, far = float(nf[0]), float(nf[1])
    return field, poses, H, W, focal, near, far


class SyntheticNeRFDataset(VolumeRenderDataset):
    def __init__(self, split="train", downsample=1.0, is_stack=False, args=None, enable_lpips=False):
        super().__init__(split, downsample, is_stack, args)
        field, poses, H, W, focal, near, far = _rig(args, "test" if split == "path" else split)
        H, W, focal = int(H / downsample), int(W / downsample), focal / downsample
        self.white_bg = bool(getattr(args, "white_bkgd", False))
        if split == "path":                     # fly-around of the box centre (or a trajectory file): poses only
            self.near_far, self.img_wh, self.focal = [near, far], (W, H), focal
            self.datadir = str(getattr(args, "datadir", ""))
            self.cxyz = ((np.array(list(args.lb)) + np.array(list(args.ub))) / 2).tolist()
            self.read_meta_path()
            self.all_rays[..., 3:6] = torch.nn.functional.normalize(self.all_rays[..., 3:6], dim=-1)
            return
        data = make_blob_dataset(field, poses, H, W, focal, near, far, white_bg=self.white_bg,
                                 n_quad=int(getattr(args, "synthetic_quadrature", 128)), normalize_dirs=True)
        self.near_far = [near, far]
        self.img_wh, self.focal, self.poses = (W, H), focal, poses
        self.image_paths = [f"synthetic_{split}_{k:04d}.png" for k in range(len(poses))]
        n_img = len(poses)
        if is_stack:
            self.all_rays = data.all_rays.view(n_img, H * W, 6)
            self.all_rgbs = data.all_rgbs.view(n_img, H * W, 3)
            self.all_idxs = data.all_idxs.view(n_img, H * W)
        else:
            self.all_rays, self.all_rgbs, self.all_idxs = data.all_rays, data.all_rgbs, data.all_idxs


class SyntheticGaussianDataset(GaussianSplattingDataset):
    def __init__(self, split="train", downsample=1.0, args=None, preload=True):
        super().__init__(split, downsample, args, preload)
        field, poses, H, W, focal, near, far = _rig(args, split)
        H, W, focal = int(H / downsample), int(W / downsample), focal / downsample
        self.white_bg = bool(getattr(args, "white_bkgd", False))
        data = make_blob_dataset(field, poses, H, W, focal, near, far, white_bg=self.white_bg,
                                 n_quad=int(getattr(args, "synthetic_quadrature", 128)), normalize_dirs=True)
        imgs = data.all_rgbs.view(len(poses), H, W, 3).permute(0, 3, 1, 2).contiguous()
        for k, pose in enumerate(poses):
            self.cameras.append(Camera.from_c2w(pose.numpy(), W, H, focal, uid=k, image=imgs[k],
                                                znear=0.01, zfar=max(100.0, 2 * far),
                                                image_name=f"synthetic_{split}_{k:04d}"))
        self.field = field
        self.compute_extent()

"""Ray generation and transforms.json readers (reference:
landmark/nerf_components/data/datasets/dataloader/utils/ray_utils.py:77-170,402-537)."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Tuple

import numpy as np
import torch


def get_ray_directions_blender(H: int, W: int, focal, center=None) -> torch.Tensor:
    """Per-pixel directions in camera space: pixel centres at +0.5, camera looks along -z."""
    fx, fy = (focal, focal) if not isinstance(focal, (list, tuple)) else focal
    cx, cy = (W / 2, H / 2) if center is None else center
    j, i = torch.meshgrid(torch.arange(H, dtype=torch.float32) + 0.5, torch.arange(W, dtype=torch.float32) + 0.5,
                          indexing="ij")
    return torch.stack(((i - cx) / fx, -(j - cy) / fy, -torch.ones_like(i)), -1)


def get_rays_with_directions(directions: torch.Tensor, c2w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    rays_d = directions @ c2w[:3, :3].T
    rays_o = c2w[:3, 3].expand(rays_d.shape)
    return rays_o.reshape(-1, 3), rays_d.reshape(-1, 3)


def get_rays(directions, c2w, camera_mode: str = "normal"):
    if camera_mode == "normal":
        return get_rays_with_directions(directions, c2w)
    # panorama: equirectangular directions over the full sphere
    H, W = directions.shape[:2]
    j, i = torch.meshgrid(torch.arange(H, dtype=torch.float32) + 0.5, torch.arange(W, dtype=torch.float32) + 0.5,
                          indexing="ij")
    theta, phi = (i / W) * 2 * math.pi - math.pi, (j / H) * math.pi - math.pi / 2
    dirs = torch.stack((torch.cos(phi) * torch.sin(theta), -torch.sin(phi), -torch.cos(phi) * torch.cos(theta)), -1)
    return get_rays_with_directions(dirs, c2w)


def pose_spherical(theta_deg: float, phi_deg: float, radius: float) -> torch.Tensor:
    """Camera on a sphere looking at the origin (NeRF-synthetic convention)."""
    def trans_t(t):
        return torch.tensor([[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, t], [0, 0, 0, 1]], dtype=torch.float32)

    def rot_phi(p):
        c, s = math.cos(p), math.sin(p)
        return torch.tensor([[1, 0, 0, 0], [0, c, -s, 0], [0, s, c, 0], [0, 0, 0, 1]], dtype=torch.float32)

    def rot_theta(t):
        c, s = math.cos(t), math.sin(t)
        return torch.tensor([[c, 0, -s, 0], [0, 1, 0, 0], [s, 0, c, 0], [0, 0, 0, 1]], dtype=torch.float32)

    c2w = rot_theta(math.radians(theta_deg)) @ rot_phi(math.radians(phi_deg)) @ trans_t(radius)
    flip = torch.tensor([[-1, 0, 0, 0], [0, 0, 1, 0], [0, 1, 0, 0], [0, 0, 0, 1]], dtype=torch.float32)
    return flip @ c2w


def load_transforms(datadir: str, split: str) -> Dict:
    with open(os.path.join(datadir, f"transforms_{split}.json"), "r", encoding="utf-8") as fh:
        return json.load(fh)


def frames_to_poses(meta: Dict) -> Tuple[List[str], np.ndarray]:
    paths = [f["file_path"] for f in meta["frames"]]
    poses = np.stack([np.array(f["transform_matrix"], dtype=np.float32) for f in meta["frames"]])
    return paths, poses


def filtering_rays(aabb: torch.Tensor, all_rays: torch.Tensor, chunk: int = 1 << 20) -> torch.Tensor:
    """Mask of rays that hit the AABB."""
    keep = []
    for s in range(0, all_rays.shape[0], chunk):
        r = all_rays[s:s + chunk]
        o, d = r[:, :3], r[:, 3:6]
        vec = torch.where(d == 0, torch.full_like(d, 1e-6), d)
        a, b = (aabb[1] - o) / vec, (aabb[0] - o) / vec
        t_min, t_max = torch.minimum(a, b).amax(-1), torch.maximum(a, b).amin(-1)
        keep.append(t_max > t_min)
    return torch.cat(keep)


def load_drone_meta(datadir: str, split: str, image_scale, subfolder=None, stride: int = 1) -> Dict:
    """Metadata of a drone capture in the ``transforms_{split}.json`` layout whose images live in
    ``images_{image_scale}/`` and whose focal length is either one ``fl_x`` for the whole capture or one per frame
    (reference: landmark/nerf_components/data/datasets/dataloader/utils/ray_utils.py:122-170).  ``subfolder`` keeps
    only frames whose parent folder is listed; ``stride`` thins the frame list (the reference's debug switch keeps
    every 50th).  Returns ``poses [N,4,4]``, ``focals`` (scalar array or ``[N]``), ``fnames``, ``hw`` (height and width
    of the first image, ``None`` when it cannot be opened) and ``imgfolder``."""
    meta = load_transforms(datadir, split)
    frames = meta["frames"]
    if subfolder:
        keep = set(subfolder)
        frames = [f for f in frames if os.path.basename(os.path.dirname(f["file_path"])) in keep]
    frames = frames[::max(int(stride), 1)]
    fnames = [f["file_path"] for f in frames]
    poses = np.stack([np.asarray(f["transform_matrix"], dtype=np.float64) for f in frames]) if frames else np.zeros((0, 4, 4))
    focals = np.asarray(meta["fl_x"]) if "fl_x" in meta else np.asarray([f["fl_x"] for f in frames])
    hw = None
    if fnames:
        for cand in (fnames[0], os.path.join(datadir, fnames[0]), os.path.join(datadir, f"images_{image_scale}", os.path.basename(fnames[0]))):
            if os.path.exists(cand):
                from PIL import Image

                with Image.open(cand) as im:
                    hw = [im.height, im.width]
                break
    return {"poses": poses, "focals": focals, "fnames": fnames, "hw": hw, "imgfolder": os.path.join(datadir, f"images_{image_scale}")}

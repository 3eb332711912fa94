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


def get_rays(directions, c2w, camera_mode="normal", *reference_tail, **reference_kw):
    """``get_rays(directions [H, W, 3], c2w, camera_mode)`` -> ``(origins [H*W, 3], directions [H*W, 3])``; in
    ``"panorama"`` mode the directions cover the full sphere (equirectangular) and only their shape is used.

    The reference's form ``get_rays(H, W, K, c2w, camera_mode="normal", offset=0.5)`` (ray_utils.py:424-469) is
    accepted as well: pixels at integer coordinates against the intrinsics ``K``, unit-length directions."""
    if isinstance(directions, int):
        H, W, K = directions, int(c2w), camera_mode
        pose = reference_tail[0] if reference_tail else reference_kw["c2w"]
        mode = reference_tail[1] if len(reference_tail) > 1 else reference_kw.get("camera_mode", "normal")
        offset = reference_tail[2] if len(reference_tail) > 2 else reference_kw.get("offset", 0.5)
        pose = torch.as_tensor(pose, dtype=torch.float32)
        j, i = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32), indexing="ij")
        if mode == "normal":
            cam = torch.stack(((i - K[0][2]) / K[0][0], -(j - K[1][2]) / K[1][1], -torch.ones_like(i)), -1)
        else:
            theta, phi = 2 * math.pi * (i + offset) / W, math.pi * (j + offset) / H
            cam = torch.stack((-torch.sin(phi) * torch.sin(theta), torch.cos(phi), torch.sin(phi) * torch.cos(theta)), -1)
        o, d = get_rays_with_directions(cam, pose)
        return o, d / d.norm(dim=-1, keepdim=True)
    if camera_mode == "normal":
        return get_rays_with_directions(directions, c2w)
    # panorama: equirectangular directions over the full sphere
    H, W = directions.shape[:2]
    j, i = torch.meshgrid(torch.arange(H, dtype=torch.float32) + 0.5, torch.arange(W, dtype=torch.float32) + 0.5,
                          indexing="ij")
    theta, phi = (i / W) * 2 * math.pi - math.pi, (j / H) * math.pi - math.pi / 2
    dirs = torch.stack((torch.cos(phi) * torch.sin(theta), -torch.sin(phi), -torch.cos(phi) * torch.cos(theta)), -1)
    return get_rays_with_directions(dirs, c2w)


def trans_t(t: float) -> torch.Tensor:
    """Translation by ``t`` along z, homogeneous ``[4, 4]``."""
    m = torch.eye(4)
    m[2, 3] = float(t)
    return m


def rot_phi(phi: float) -> torch.Tensor:
    """Rotation by ``phi`` radians about x, homogeneous ``[4, 4]``."""
    c, s = math.cos(phi), math.sin(phi)
    return torch.tensor([[1, 0, 0, 0], [0, c, -s, 0], [0, s, c, 0], [0, 0, 0, 1]], dtype=torch.float32)


def rot_theta(theta: float) -> torch.Tensor:
    """Rotation by ``theta`` radians about y (NeRF-synthetic sign), homogeneous ``[4, 4]``."""
    c, s = math.cos(theta), math.sin(theta)
    return torch.tensor([[c, 0, -s, 0], [0, 1, 0, 0], [s, 0, c, 0], [0, 0, 0, 1]], dtype=torch.float32)


def pose_spherical(theta_deg: float, phi_deg: float, radius: float, zval=None) -> torch.Tensor:
    """Camera on a sphere looking at the origin (NeRF-synthetic convention); ``zval`` overrides the camera height."""
    c2w = rot_theta(math.radians(theta_deg)) @ rot_phi(math.radians(phi_deg)) @ trans_t(radius)
    flip = torch.tensor([[-1, 0, 0, 0], [0, 0, 1, 0], [0, 1, 0, 0], [0, 0, 0, 1]], dtype=torch.float32)
    c2w = flip @ c2w
    if zval is not None:
        c2w[2, 3] = float(zval)
    return c2w


def get_ray_directions(H: int, W: int, focal, center=None) -> torch.Tensor:
    """Per-pixel directions ``[H, W, 3]`` of a camera that looks along +z with y down (OpenCV axes), pixel ``(i, j)``
    at integer coordinates, not normalised (reference: ray_utils.py:473-491)."""
    fx, fy = (focal, focal) if not isinstance(focal, (list, tuple)) else focal
    cx, cy = (W / 2, H / 2) if center is None else center
    j, i = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32), indexing="ij")
    return torch.stack(((i - cx) / fx, (j - cy) / fy, torch.ones_like(i)), -1)


def depth2dist(z_vals: torch.Tensor, cos_angle: torch.Tensor) -> torch.Tensor:
    """Sample spacings along the ray from depths along the optical axis: differences of ``z_vals [..., S]`` (the last
    one open-ended, 1e10) scaled by ``cos_angle [...]``, the per-ray ratio of ray length to depth."""
    gaps = torch.diff(z_vals, dim=-1)
    last = torch.full_like(z_vals[..., :1], 1e10)
    return torch.cat((gaps, last), dim=-1) * cos_angle[..., None]


def patchify(img: torch.Tensor, rays_o: torch.Tensor, rays_d: torch.Tensor, H: int, W: int, ps: int):
    """Cut an image and its rays into non-overlapping ``ps x ps`` patches (incomplete border patches are dropped):
    returns ``(rgb [n, ps*ps, 3], rays [n, ps*ps, 6])`` with patches in row-major order."""
    def cut(t):
        t = t.reshape(H, W, 3)[:H // ps * ps, :W // ps * ps]
        return t.reshape(H // ps, ps, W // ps, ps, 3).permute(0, 2, 1, 3, 4).reshape(-1, ps * ps, 3)

    return cut(img), torch.cat((cut(rays_o), cut(rays_d)), dim=-1)


def listify_matrix(matrix) -> List[list]:
    """Rows of a matrix as plain lists (for JSON)."""
    return [list(row) for row in matrix]


def read_Image(f_path: str, transform=None) -> torch.Tensor:
    """RGB image as ``[H*W, 3]`` floats in [0, 1]; ``transform`` (a PIL -> ``[3, H, W]`` tensor callable) is optional."""
    from PIL import Image

    with Image.open(f_path) as im:
        im = im.convert("RGB")
        chw = transform(im) if transform is not None else torch.from_numpy(
            np.asarray(im, dtype=np.float32) / 255.0).permute(2, 0, 1)
    return chw.reshape(3, -1).permute(1, 0).contiguous()


def load_json_render_path(pathfolder: str, posefile: str, render_skip: int = 1) -> np.ndarray:
    """Camera-to-world matrices of every ``render_skip``-th frame of a trajectory file."""
    assert posefile.endswith("json"), "trajectory files are JSON"
    with open(os.path.join(pathfolder, posefile), "r", encoding="utf-8") as fh:
        frames = json.load(fh)["frames"][::max(int(render_skip), 1)]
    return np.array([f["transform_matrix"] for f in frames])


def pad_poses(p: np.ndarray) -> np.ndarray:
    """``[..., 3, 4]`` -> ``[..., 4, 4]`` with the homogeneous bottom row."""
    bottom = np.broadcast_to(np.array([0.0, 0.0, 0.0, 1.0]), p[..., :1, :4].shape)
    return np.concatenate((p[..., :3, :4], bottom), axis=-2)


def unpad_poses(p: np.ndarray) -> np.ndarray:
    return p[..., :3, :4]


def transform_poses_pca(poses: np.ndarray):
    """Re-express camera-to-world poses ``[N, 3|4, 4]`` in the principal axes of the camera positions (largest spread
    along x, smallest along z), centred on their mean, flipped so that the cameras' y axes point up on average, and
    scaled so that the positions fit in [-1, 1]^3.  Returns ``(poses [N, 3, 4], transform [4, 4])`` where
    ``transform`` maps old world coordinates to new ones."""
    centres = poses[:, :3, 3]
    mean = centres.mean(axis=0)
    spread = centres - mean
    eigval, eigvec = np.linalg.eigh(spread.T @ spread)           # ascending eigenvalues of a symmetric matrix
    rot = eigvec[:, ::-1].T
    if np.linalg.det(rot) < 0:
        rot = np.diag([1.0, 1.0, -1.0]) @ rot
    transform = np.eye(4)
    transform[:3, :3], transform[:3, 3] = rot, rot @ -mean
    out = unpad_poses(transform @ pad_poses(poses))
    if out.mean(axis=0)[2, 1] < 0:                                # cameras upside down on average
        flip = np.diag([1.0, -1.0, -1.0, 1.0])
        out, transform = flip[:3, :3] @ out, flip @ transform
    scale = 1.0 / np.max(np.abs(out[:, :3, 3]))
    out[:, :3, 3] *= scale
    transform = np.diag([scale, scale, scale, 1.0]) @ transform
    return out, transform


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

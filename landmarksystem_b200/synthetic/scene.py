"""Analytic synthetic scenes: a Gaussian-blob density/colour field, pinhole camera rigs, ray
generation and ground-truth compositing.  They stand in for the MatrixCity data the reference's
tests depend on, with the same ray conventions (pixel centres at +0.5, camera looks along -z,
``rays_d = dir @ R^T``; reference: landmark/nerf_components/data/datasets/dataloader/utils/
ray_utils.py:494-537).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch


@dataclass
class BlobField:
    """Sum of isotropic Gaussian blobs: ``sigma(x) = sum_i peak_i * exp(-|x - c_i|^2 / (2 s_i^2))``;
    colour is the density-weighted mean of the blob colours."""

    centers: torch.Tensor   # [K, 3]
    scales: torch.Tensor    # [K]
    peaks: torch.Tensor     # [K]
    colors: torch.Tensor    # [K, 3]

    @staticmethod
    def random(n_blobs: int, lb: Sequence[float], ub: Sequence[float], seed: int = 0, margin: float = 0.1,
               scale_range=(0.05, 0.2), peak_range=(5.0, 50.0)) -> "BlobField":
        g = torch.Generator().manual_seed(seed)
        lb_t, ub_t = torch.tensor(lb, dtype=torch.float32), torch.tensor(ub, dtype=torch.float32)
        ext = ub_t - lb_t
        lo, hi = lb_t + margin * ext, ub_t - margin * ext
        centers = lo + (hi - lo) * torch.rand(n_blobs, 3, generator=g)
        unit = ext.min() / 2.0  # scale ranges are given for a [-1, 1]^3 box
        scales = (scale_range[0] + (scale_range[1] - scale_range[0]) * torch.rand(n_blobs, generator=g)) * unit
        peaks = (peak_range[0] + (peak_range[1] - peak_range[0]) * torch.rand(n_blobs, generator=g)) / unit
        colors = torch.rand(n_blobs, 3, generator=g)
        return BlobField(centers, scales, peaks, colors)

    def to(self, device) -> "BlobField":
        return BlobField(self.centers.to(device), self.scales.to(device), self.peaks.to(device),
                         self.colors.to(device))

    def query(self, xyz: torch.Tensor, chunk: int = 1 << 16) -> Tuple[torch.Tensor, torch.Tensor]:
        """``xyz [N, 3]`` -> ``(sigma [N], rgb [N, 3])``."""
        sig, rgb = [], []
        for s in range(0, xyz.shape[0], chunk):
            x = xyz[s:s + chunk]
            d2 = ((x[:, None, :] - self.centers[None]) ** 2).sum(-1)
            w = self.peaks[None] * torch.exp(-d2 / (2.0 * self.scales[None] ** 2))
            total = w.sum(-1)
            sig.append(total)
            rgb.append((w @ self.colors) / total.clamp_min(1e-12)[:, None])
        return torch.cat(sig), torch.cat(rgb)

    @torch.no_grad()
    def render(self, rays_o: torch.Tensor, rays_d: torch.Tensor, near: float, far: float, n_samples: int = 192,
               white_bg: bool = False, chunk: int = 4096) -> torch.Tensor:
        """Ground-truth pixels by dense quadrature along each ray."""
        out = []
        t = torch.linspace(near, far, n_samples, device=rays_o.device)
        delta = (far - near) / (n_samples - 1)
        for s in range(0, rays_o.shape[0], chunk):
            o, d = rays_o[s:s + chunk], rays_d[s:s + chunk]
            pts = o[:, None, :] + d[:, None, :] * t[None, :, None]
            sigma, rgb = self.query(pts.reshape(-1, 3))
            sigma, rgb = sigma.view(-1, n_samples), rgb.view(-1, n_samples, 3)
            alpha = 1.0 - torch.exp(-sigma * delta * d.norm(dim=-1, keepdim=True))
            trans = torch.cumprod(torch.cat((torch.ones_like(alpha[:, :1]), 1.0 - alpha + 1e-10), -1), -1)[:, :-1]
            w = alpha * trans
            pix = (w[..., None] * rgb).sum(1)
            if white_bg:
                pix = pix + (1.0 - w.sum(-1, keepdim=True))
            out.append(pix.clamp(0, 1))
        return torch.cat(out)


def look_at(eye: torch.Tensor, target: torch.Tensor, up=(0.0, 0.0, 1.0)) -> torch.Tensor:
    """Camera-to-world ``[4, 4]`` in the OpenGL convention (camera looks along -z, +y up)."""
    fwd = target - eye
    fwd = fwd / fwd.norm()
    upv = torch.tensor(up, dtype=torch.float32)
    right = torch.linalg.cross(fwd, upv)
    if right.norm() < 1e-6:
        right = torch.linalg.cross(fwd, torch.tensor([0.0, 1.0, 0.0]))
    right = right / right.norm()
    true_up = torch.linalg.cross(right, fwd)
    c2w = torch.eye(4)
    c2w[:3, 0], c2w[:3, 1], c2w[:3, 2], c2w[:3, 3] = right, true_up, -fwd, eye
    return c2w


def ring_cameras(n: int, radius: float, height: float = 0.0, target=(0.0, 0.0, 0.0)) -> torch.Tensor:
    """``n`` cameras on a horizontal ring looking at ``target`` -> ``[n, 4, 4]``."""
    tgt = torch.tensor(target, dtype=torch.float32)
    poses = []
    for i in range(n):
        a = 2.0 * math.pi * i / n
        eye = torch.tensor([radius * math.cos(a), radius * math.sin(a), height])
        poses.append(look_at(eye, tgt))
    return torch.stack(poses)


def aerial_cameras(n: int, lb: Sequence[float], ub: Sequence[float], altitude: float, max_tilt_deg: float = 30.0,
                   seed: int = 0) -> torch.Tensor:
    """``n`` nadir-ish cameras over the box footprint at ``altitude`` above ``lb_z`` with random tilt."""
    g = torch.Generator().manual_seed(seed)
    poses = []
    for _ in range(n):
        u = torch.rand(2, generator=g)
        eye = torch.tensor([lb[0] + (ub[0] - lb[0]) * float(u[0]), lb[1] + (ub[1] - lb[1]) * float(u[1]),
                            lb[2] + altitude])
        tilt = math.radians(max_tilt_deg) * float(torch.rand((), generator=g))
        az = 2.0 * math.pi * float(torch.rand((), generator=g))
        off = math.tan(tilt) * altitude
        tgt = torch.tensor([eye[0] + off * math.cos(az), eye[1] + off * math.sin(az), lb[2]])
        poses.append(look_at(eye, tgt, up=(0.0, 1.0, 0.0)))
    return torch.stack(poses)


def camera_rays(c2w: torch.Tensor, H: int, W: int, focal: float, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """All ``H*W`` rays of one camera: ``(origins [HW, 3], un-normalised directions [HW, 3])``."""
    device = device or c2w.device
    j, i = torch.meshgrid(torch.arange(H, device=device, dtype=torch.float32) + 0.5,
                          torch.arange(W, device=device, dtype=torch.float32) + 0.5, indexing="ij")
    dirs = torch.stack(((i - W / 2) / focal, -(j - H / 2) / focal, -torch.ones_like(i)), -1)
    c2w = c2w.to(device)
    rays_d = dirs.reshape(-1, 3) @ c2w[:3, :3].T
    rays_o = c2w[:3, 3].expand_as(rays_d)
    return rays_o.contiguous(), rays_d.contiguous()


@dataclass
class SyntheticNeRFData:
    """Flat training set: ``all_rays [N, 6]``, ``all_rgbs [N, 3]``, ``all_idxs [N]`` (+ per-image views)."""

    all_rays: torch.Tensor
    all_rgbs: torch.Tensor
    all_idxs: torch.Tensor
    poses: torch.Tensor
    H: int
    W: int
    focal: float
    near_far: Tuple[float, float]


def make_blob_dataset(field: BlobField, poses: torch.Tensor, H: int, W: int, focal: float, near: float, far: float,
                      white_bg: bool = False, n_quad: int = 192, device="cpu",
                      normalize_dirs: bool = False) -> SyntheticNeRFData:
    rays, rgbs, idxs = [], [], []
    f = field.to(device)
    for k, pose in enumerate(poses):
        o, d = camera_rays(pose, H, W, focal, device)
        if normalize_dirs:
            d = d / d.norm(dim=-1, keepdim=True)
        rays.append(torch.cat((o, d), -1).cpu())
        rgbs.append(f.render(o, d, near, far, n_quad, white_bg).cpu())
        idxs.append(torch.full((H * W,), float(k)))
    return SyntheticNeRFData(torch.cat(rays), torch.cat(rgbs), torch.cat(idxs), poses, H, W, focal, (near, far))

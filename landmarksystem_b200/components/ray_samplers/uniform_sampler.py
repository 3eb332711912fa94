"""Uniform / hull sampling of points along rays (reference:
landmark/nerf_components/ray_samplers/uniform_sampler.py:42-98).

Dense mode: ``z_k = t_min + step * (k + u)`` with ``t_min`` the ray's AABB entry clamped to
``[near, far]`` and one jitter ``u`` per ray while training.  Hull mode (used at render time):
``n`` samples linearly spaced from ``near`` to the ground-plane hit ``-(o_z - lb_z) / d_z`` (``far``
for rays that look up), stratified while training.  Device-agnostic: the reference hard-codes
``.cuda()`` in the hull branch; this implementation follows the rays' device.
"""
from __future__ import annotations

from typing import Union

import torch

from ..data.rays import Rays
from ..data.samples import Samples
from .base_sampler import BaseSampler


class UniformSampler(BaseSampler):
    def __init__(self, num_samples=None, step_size=None, aabb=None, near_far=None):
        super().__init__(num_samples)
        self.step_size = step_size
        self.aabb = aabb
        self.near_far = near_far
        self.save_init_kwargs(locals())

    def compute_z_vals(self, rays_data: torch.Tensor, num_samples: int, random_sampling: bool,
                       sample_within_hull: bool) -> torch.Tensor:
        origin, dirs = rays_data[..., :3], rays_data[..., 3:6]
        near, far = float(self.near_far[0]), float(self.near_far[1])
        aabb = self.aabb.to(rays_data.device)
        if not sample_within_hull:
            safe = torch.where(dirs == 0, torch.full_like(dirs, 1e-6), dirs)
            t_min = torch.minimum((aabb[1] - origin) / safe, (aabb[0] - origin) / safe).amax(-1).clamp(near, far)
            k = torch.arange(num_samples, device=rays_data.device, dtype=torch.float32)[None]
            if random_sampling:
                k = k + torch.rand(origin.shape[0], 1, device=rays_data.device)
            return t_min[:, None] + float(self.step_size) * k
        o_z = origin[:, 2:3] - aabb[0, 2]
        d_z = dirs[:, 2:3]
        hit = -(o_z / torch.where(d_z == 0, torch.full_like(d_z, 1e-6), d_z))
        hit = torch.where(d_z >= 0, torch.full_like(hit, far), hit)
        t = torch.linspace(0.0, 1.0, num_samples, device=rays_data.device)
        z = near * (1.0 - t) + hit * t
        if random_sampling:
            mids = 0.5 * (z[:, 1:] + z[:, :-1])
            upper = torch.cat((mids, z[:, -1:]), -1)
            lower = torch.cat((z[:, :1], mids), -1)
            z = lower + (upper - lower) * torch.rand_like(z)
        return z

    def forward(self, rays: Union[Rays, torch.Tensor], num_samples: int = -1, random_sampling: bool = True,
                sample_within_hull: bool = False):
        """Returns ``(Samples [R, S], inside-AABB mask [R, S])``."""
        data = rays.data if isinstance(rays, Rays) else rays
        n = num_samples if num_samples > 0 else self.num_samples
        z = self.compute_z_vals(data, n, random_sampling, sample_within_hull)
        origin, dirs = data[..., :3], data[..., 3:6]
        xyz = origin[:, None, :] + dirs[:, None, :] * z[..., None]
        cam = data[..., 6:7].expand(-1, n) if data.shape[-1] > 6 else None
        samples = Samples(xyz=xyz, dirs=dirs[:, None, :].expand_as(xyz), z_vals=z, camera_idx=cam,
                          rank=getattr(rays, "rank", None), group=getattr(rays, "group", None))
        aabb = self.aabb.to(data.device)
        inside = ~((xyz < aabb[0]) | (xyz > aabb[1])).any(dim=-1)
        return samples, inside


class FusedUniformSampler(UniformSampler):
    """Kernel-runtime name of the sampler.  The reference ships only a stub that raises
    (landmark/nerf_components/ray_samplers/fused_uniform_sampler.py:10-29); here it is the same
    sampler, whose output feeds the fused field kernels."""

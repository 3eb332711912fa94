"""Occupancy-grid sampler (reference: landmark/nerf_components/ray_samplers/volumetric_sampler.py:57-119).

The reference marches with nerfacc into packed arrays and re-pads them to ``[R, max_n]`` with a host
sync on the maximum count; here the marching kernel writes the padded layout directly."""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..data.rays import Rays
from ..data.samples import Samples
from .base_sampler import BaseSampler


class VolumetricSampler(BaseSampler):
    def __init__(self, occupancy_grid=None, density_fn: Optional[Callable] = None, near_far=(0.0, 1e10),
                 step_size: float = 1e-3, alpha_thre: float = 0.01, cone_angle: float = 0.004, max_samples: int = 256):
        super().__init__()
        self.occupancy_grid = occupancy_grid
        self.density_fn = density_fn
        self.near_far, self.step_size = near_far, step_size
        self.alpha_thre, self.cone_angle, self.max_samples = alpha_thre, cone_angle, max_samples
        self.save_init_kwargs(locals())

    def get_sigma_fn(self, origins, directions):
        if self.density_fn is None or not self.training:
            return None

        def sigma_fn(t_starts, t_ends, ray_indices):
            mid = 0.5 * (t_starts + t_ends)[:, None]
            return self.density_fn(origins[ray_indices] + directions[ray_indices] * mid).reshape(-1)

        # a field may evaluate the marched samples straight from the padded [R, S] interval block (sample index ->
        # position -> density with its own kernels) instead of receiving gathered positions
        from_samples = getattr(self.density_fn, "from_samples", None)
        if from_samples is not None:
            sigma_fn.from_samples = lambda idx, S, ts, te: from_samples(idx, S, origins, directions, ts, te)
        return sigma_fn

    @torch.no_grad()
    def forward(self, ray_bundle, training: bool = True, render_stratified_sampling: bool = True,
                near_plane: Optional[float] = None, far_plane: Optional[float] = None, lean: bool = False):
        """``lean``: return ``(origins, directions, t_starts, t_ends, valid)`` instead of packed sample records - a caller
        that only evaluates the valid samples builds their positions itself and never materialises the ``[R, S, 13]`` block."""
        data = ray_bundle.data if isinstance(ray_bundle, Rays) else ray_bundle
        o, d = data[:, :3].contiguous(), data[:, 3:6].contiguous()
        near = self.near_far[0] if near_plane is None else near_plane
        far = self.near_far[1] if far_plane is None else far_plane
        counts, ts, te = self.occupancy_grid.sampling(
            o, d, sigma_fn=self.get_sigma_fn(o, d), near_plane=near, far_plane=far, render_step_size=self.step_size,
            stratified=training or render_stratified_sampling, cone_angle=self.cone_angle,
            alpha_thre=self.alpha_thre if training else 0.0, max_samples=self.max_samples)
        S = ts.shape[1]
        valid = torch.arange(S, device=data.device)[None] < counts[:, None]
        if lean:
            return o, d, ts, te, valid
        z = 0.5 * (ts + te)
        xyz = o[:, None, :] + d[:, None, :] * z[..., None]
        cam = data[:, 6:7].expand(-1, S) if data.shape[1] > 6 else None
        samples = Samples(xyz=xyz, dirs=d[:, None, :].expand_as(xyz), z_vals=z, camera_idx=cam,
                          rank=getattr(ray_bundle, "rank", None), group=getattr(ray_bundle, "group", None))
        samples.t_starts, samples.t_ends = ts, te
        return samples, valid

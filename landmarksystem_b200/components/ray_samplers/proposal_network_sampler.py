"""Proposal-network sampling for Nerfacto (reference:
landmark/nerf_components/ray_samplers/proposal_network_sampler.py:20-501).

Rays are first sampled uniformly in a normalised "spacing" coordinate ``s`` in ``[0, 1]`` whose map
to distance is linear for near range and in disparity beyond (``f(x) = x/2`` for ``x < 1`` else
``1 - 1/(2x)``).  Small hash-grid density networks ("proposal networks") then provide histograms from
which finer sample sets are drawn by inverse-CDF sampling; the weights are annealed (``w^a``) early in
training and the proposal networks receive gradients only every few steps.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch import nn

from ...ops import composite_weights
from ..fields.encodings.hash_encoding import HashEncoding
from ..fields.mlp_decoder import MLPDecoder
from ..model.base_module import BaseModule
from ..utils.activation_utils import trunc_exp
from .base_sampler import BaseSampler


@dataclass
class RaySamples:
    """Intervals along rays: Euclidean ``starts/ends [R, S, 1]`` and normalised ``spacing_*`` in [0, 1]."""
    origins: torch.Tensor
    directions: torch.Tensor
    starts: torch.Tensor
    ends: torch.Tensor
    spacing_starts: torch.Tensor
    spacing_ends: torch.Tensor
    spacing_to_euclidean_fn: Optional[Callable] = None
    camera_indices: Optional[torch.Tensor] = None

    @property
    def positions(self) -> torch.Tensor:
        mid = 0.5 * (self.starts + self.ends)
        return self.origins[:, None, :] + self.directions[:, None, :] * mid

    @property
    def deltas(self) -> torch.Tensor:
        return self.ends - self.starts

    def get_weights(self, densities: torch.Tensor) -> torch.Tensor:
        """``densities [R, S, 1]`` -> weights ``[R, S, 1]``."""
        w, _ = composite_weights(densities[..., 0].float(), self.deltas[..., 0].contiguous())
        return torch.nan_to_num(w)[..., None]


def spacing_fn(x):
    return torch.where(x < 1, x / 2, 1 - 1 / (2 * x))


def spacing_fn_inv(x):
    return torch.where(x < 0.5, 2 * x, 1 / (2 - 2 * x))


class SpacedSampler(BaseSampler):
    """Uniform bins in spacing space with optional stratified jitter."""

    def __init__(self, num_samples: Optional[int] = None, train_stratified: bool = True, single_jitter: bool = False):
        super().__init__(num_samples)
        self.train_stratified, self.single_jitter = train_stratified, single_jitter

    def forward(self, origins, directions, near, far, num_samples: Optional[int] = None, camera_indices=None):
        n = num_samples or self.num_samples
        R, dev = origins.shape[0], origins.device
        bins = torch.linspace(0.0, 1.0, n + 1, device=dev)[None].expand(R, -1)
        if self.train_stratified and self.training:
            t_rand = torch.rand((R, 1) if self.single_jitter else (R, n + 1), device=dev)
            centers = 0.5 * (bins[:, 1:] + bins[:, :-1])
            upper = torch.cat((centers, bins[:, -1:]), -1)
            lower = torch.cat((bins[:, :1], centers), -1)
            bins = lower + (upper - lower) * t_rand
        s_near, s_far = spacing_fn(torch.as_tensor(float(near), device=dev)), spacing_fn(torch.as_tensor(float(far), device=dev))

        def to_euclid(s):
            return spacing_fn_inv(s * s_far + (1 - s) * s_near)

        eu = to_euclid(bins)
        return RaySamples(origins, directions, eu[:, :-1, None], eu[:, 1:, None], bins[:, :-1, None], bins[:, 1:, None],
                          to_euclid, camera_indices)


class PropPDFSampler(BaseSampler):
    """Resample ``num_samples`` intervals from a histogram over existing intervals."""

    def __init__(self, num_samples: Optional[int] = None, train_stratified: bool = True, single_jitter: bool = False,
                 include_original: bool = True, histogram_padding: float = 0.01):
        super().__init__(num_samples)
        self.train_stratified, self.single_jitter = train_stratified, single_jitter
        self.include_original, self.histogram_padding = include_original, histogram_padding

    def forward(self, ray_samples: RaySamples, weights: torch.Tensor, num_samples: Optional[int] = None, eps: float = 1e-5):
        n = num_samples or self.num_samples
        num_bins = n + 1
        existing = torch.cat((ray_samples.spacing_starts[..., 0], ray_samples.spacing_ends[..., -1:, 0]), -1)
        dev = existing.device
        lead = existing.shape[:-1]
        if self.train_stratified and self.training:
            u = torch.linspace(0.0, 1.0 - 1.0 / num_bins, num_bins, device=dev).expand(*lead, num_bins)
            rand = torch.rand((*lead, 1 if self.single_jitter else num_bins), device=dev) / num_bins
            u = u + rand
        else:
            u = torch.linspace(0.0, 1.0 - 1.0 / num_bins, num_bins, device=dev) + 1.0 / (2 * num_bins)
            u = u.expand(*lead, num_bins)
        u = u.contiguous()
        bins = None
        if existing.is_cuda and existing.dim() == 2 and max(existing.shape[-1], num_bins) <= 1025:
            from ...ops import native
            from ...ops.pdf import prop_resample

            if native.available():       # histogram, CDF, inverse-CDF search and ordered merge in one warp-per-ray kernel
                bins = prop_resample(weights[..., 0], existing, u, self.histogram_padding, eps, self.include_original)
        if bins is None:
            bins = self._resample_torch(weights, existing, u, eps)
        eu = ray_samples.spacing_to_euclidean_fn(bins)
        return RaySamples(ray_samples.origins, ray_samples.directions, eu[:, :-1, None], eu[:, 1:, None],
                          bins[:, :-1, None], bins[:, 1:, None], ray_samples.spacing_to_euclidean_fn,
                          ray_samples.camera_indices)

    # the same computation with PyTorch ops (CPU, or shapes beyond the kernel's shared-memory window)
    def _resample_torch(self, weights, existing, u, eps):
        w = weights[..., 0] + self.histogram_padding
        w_sum = w.sum(-1, keepdim=True)
        padding = torch.relu(eps - w_sum)
        w = w + padding / w.shape[-1]
        w_sum = w_sum + padding
        pdf = w / w_sum
        cdf = torch.cat((torch.zeros_like(pdf[..., :1]), torch.cumsum(pdf, -1).clamp(max=1.0)), -1)
        inds = torch.searchsorted(cdf, u, side="right")
        below = (inds - 1).clamp(0, existing.shape[-1] - 1)
        above = inds.clamp(0, existing.shape[-1] - 1)
        cdf0, cdf1 = torch.gather(cdf, -1, below), torch.gather(cdf, -1, above)
        b0, b1 = torch.gather(existing, -1, below), torch.gather(existing, -1, above)
        t = torch.clip(torch.nan_to_num((u - cdf0) / (cdf1 - cdf0), 0), 0, 1)
        bins = (b0 + t * (b1 - b0)).detach()
        if self.include_original:
            bins, _ = torch.sort(torch.cat((existing, bins), -1), -1)
        return bins


class HashMLPDensityField(BaseModule):
    """Small hash grid + MLP density network used as a proposal network."""

    def __init__(self, aabb, num_levels: int = 5, max_res: int = 128, base_res: int = 16, log2_hashmap_size: int = 17,
                 features_per_level: int = 2, hidden_dim: int = 16, num_layers: int = 2, spatial_distortion=None,
                 device="cpu"):
        super().__init__()
        self.register_buffer("aabb", torch.as_tensor(aabb, dtype=torch.float32))
        self.spatial_distortion = spatial_distortion
        self.encoding = HashEncoding(num_levels, base_res, max_res, log2_hashmap_size, features_per_level, device=device)
        self.mlp = MLPDecoder(self.encoding.get_out_dim(), hidden_dim, num_layers, 1, None, mlp_bias=False).to(device)
        self.save_init_kwargs(locals())

    def density_fn(self, positions: torch.Tensor) -> torch.Tensor:
        shape = positions.shape[:-1]
        if self.spatial_distortion is not None:
            pos = (self.spatial_distortion(positions) + 2.0) / 4.0
        else:
            pos = (positions - self.aabb[0]) / (self.aabb[1] - self.aabb[0])
        inside = ((pos > 0.0) & (pos < 1.0)).all(dim=-1)
        pos = (pos * inside[..., None]).reshape(-1, 3)
        raw = self.mlp(self.encoding(pos)).float().view(*shape, 1)
        return trunc_exp(raw) * inside[..., None]

    forward = density_fn


def contract(x: torch.Tensor) -> torch.Tensor:
    """L-infinity scene contraction: identity inside the unit cube, ``(2 - 1/|x|) x / |x|`` outside."""
    mag = x.abs().amax(dim=-1, keepdim=True).clamp_min(1e-9)
    return torch.where(mag < 1, x, (2 - 1 / mag) * (x / mag))


class ProposalNetworks(nn.Module):
    def __init__(self, aabb, num_proposal_iterations: int = 2, proposal_net_args_list: Sequence[dict] = (),
                 use_same_proposal_network: bool = False, spatial_distortion=None, device="cpu"):
        super().__init__()
        n = 1 if use_same_proposal_network else num_proposal_iterations
        nets = []
        for i in range(n):
            args = dict(proposal_net_args_list[min(i, len(proposal_net_args_list) - 1)]) if proposal_net_args_list else {}
            nets.append(HashMLPDensityField(aabb, spatial_distortion=spatial_distortion, device=device, **args))
        self.networks = nn.ModuleList(nets)
        self.density_fns = [self.networks[0 if use_same_proposal_network else i].density_fn
                            for i in range(num_proposal_iterations)]

    def density_fn(self, positions: torch.Tensor, level: int = 0) -> torch.Tensor:
        """Density of proposal level ``level`` at ``positions``."""
        return self.density_fns[level](positions)

    def get_density(self, positions: torch.Tensor, level: int = 0) -> torch.Tensor:
        return self.density_fn(positions, level)


class ProposalNetworkSampler(BaseSampler):
    def __init__(self, num_proposal_samples_per_ray: Tuple[int, ...] = (256, 96), num_nerf_samples_per_ray: int = 48,
                 num_proposal_network_iterations: int = 2, single_jitter: bool = False,
                 update_sched: Callable[[int], int] = lambda x: 1, proposal_weights_anneal_max_num_iters: int = 1000,
                 proposal_weights_anneal_slope: float = 10.0, use_proposal_weight_anneal: bool = True):
        super().__init__()
        assert num_proposal_network_iterations >= 1
        self.num_proposal_samples_per_ray = tuple(num_proposal_samples_per_ray)
        self.num_nerf_samples_per_ray = num_nerf_samples_per_ray
        self.num_proposal_network_iterations = num_proposal_network_iterations
        self.update_sched = update_sched
        self.anneal_iters, self.anneal_slope = proposal_weights_anneal_max_num_iters, proposal_weights_anneal_slope
        self.use_anneal = use_proposal_weight_anneal
        self.initial_sampler = SpacedSampler(single_jitter=single_jitter)
        self.pdf_sampler = PropPDFSampler(include_original=False, single_jitter=single_jitter)
        self._anneal, self._steps_since_update, self._step = 1.0, 0, 0

    def set_anneal(self, anneal: float) -> None:
        self._anneal = anneal

    def step_cb(self, step: int) -> None:
        """Call once per training iteration before sampling."""
        self._step = step
        self._steps_since_update += 1
        if self.use_anneal:
            frac = float(np.clip(step / max(self.anneal_iters, 1), 0, 1))
            b = self.anneal_slope
            self._anneal = b * frac / ((b - 1) * frac + 1)

    def forward(self, origins, directions, near, far, density_fns: List[Callable], camera_indices=None,
                render_stratified_sampling: bool = False):
        """Returns ``(ray_samples, weights_list, ray_samples_list)``.  ``render_stratified_sampling`` keeps the
        jitter of the bins outside training as well (reference: proposal_network_sampler.py:184-199)."""
        stratified = bool(self.training or render_stratified_sampling)
        self.initial_sampler.train(stratified)
        self.pdf_sampler.train(stratified)
        weights_list, samples_list = [], []
        n = self.num_proposal_network_iterations
        weights = ray_samples = None
        updated = self._steps_since_update > self.update_sched(self._step) or self._step < 10
        for level in range(n + 1):
            is_prop = level < n
            num = self.num_proposal_samples_per_ray[level] if is_prop else self.num_nerf_samples_per_ray
            if level == 0:
                ray_samples = self.initial_sampler(origins, directions, near, far, num, camera_indices)
            else:
                ray_samples = self.pdf_sampler(ray_samples, torch.pow(weights, self._anneal), num)
            if is_prop:
                if updated and self.training:
                    density = density_fns[level](ray_samples.positions)
                else:
                    with torch.no_grad():
                        density = density_fns[level](ray_samples.positions)
                weights = ray_samples.get_weights(density)
                weights_list.append(weights)
                samples_list.append(ray_samples)
        if updated:
            self._steps_since_update = 0
        return ray_samples, weights_list, samples_list

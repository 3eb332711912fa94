"""Inverse-CDF importance resampling along rays (reference:
landmark/nerf_components/ray_samplers/pdf_sampler.py:37-116).

The new samples are drawn from the piecewise-constant PDF defined by ``weights`` over the bins
between sample mid-points, then merged (sorted) with the existing ``z_vals``.  The reference
computes the bin edges as half the *difference* of neighbouring samples; the mid-point (half the
sum) is used here, which is what the inverse-CDF construction requires.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from ..data.rays import Rays
from ..data.samples import Samples
from .base_sampler import BaseSampler


def sample_pdf(bins: torch.Tensor, weights: torch.Tensor, n_samples: int, det: bool = False) -> torch.Tensor:
    """``bins [R, B+1]`` edges, ``weights [R, B]`` -> ``[R, n_samples]`` positions (no gradient on CUDA: the
    callers detach the result).  CUDA inputs go through one kernel (``ops/csrc/pdf.cu``)."""
    if weights.is_cuda and weights.dim() == 2 and not (weights.requires_grad and torch.is_grad_enabled()) \
            and 2 * (weights.shape[-1] + 1) * 4 <= 48 * 1024:
        from ...ops.pdf import pdf_resample

        u = None if det else torch.rand(weights.shape[0], n_samples, device=weights.device)
        return pdf_resample(bins, weights, n_samples, u)
    weights = weights + 1e-5
    pdf = weights / weights.sum(-1, keepdim=True)
    cdf = torch.cat((torch.zeros_like(pdf[..., :1]), torch.cumsum(pdf, -1)), -1)
    if det:
        u = torch.linspace(0.0, 1.0, n_samples, device=weights.device).expand(*cdf.shape[:-1], n_samples)
    else:
        u = torch.rand(*cdf.shape[:-1], n_samples, device=weights.device)
    u = u.contiguous()
    inds = torch.searchsorted(cdf.detach(), u, right=True)
    below = (inds - 1).clamp(min=0)
    above = inds.clamp(max=cdf.shape[-1] - 1)
    cdf_lo, cdf_hi = torch.gather(cdf, -1, below), torch.gather(cdf, -1, above)
    bin_lo, bin_hi = torch.gather(bins, -1, below), torch.gather(bins, -1, above)
    denom = cdf_hi - cdf_lo
    denom = torch.where(denom < 1e-5, torch.ones_like(denom), denom)
    return bin_lo + (u - cdf_lo) / denom * (bin_hi - bin_lo)


class PDFSampler(BaseSampler):
    def __init__(self, num_samples: Optional[int] = None):
        super().__init__(num_samples)
        self.save_init_kwargs(locals())

    def forward(self, rays: Union[Rays, torch.Tensor], z_vals: torch.Tensor, weights: torch.Tensor,
                num_samples: Optional[int] = None, det: bool = False) -> Samples:
        """``weights`` are the interior weights ``w[..., 1:-1]`` of the coarse pass."""
        data = rays.data if isinstance(rays, Rays) else rays
        n = self.num_samples if num_samples is None else num_samples
        mids = 0.5 * (z_vals[..., 1:] + z_vals[..., :-1])
        z_new = sample_pdf(mids, weights, n, det).detach()
        z_all, _ = torch.sort(torch.cat((z_vals, z_new), -1), -1)
        origin, dirs = data[..., :3], data[..., 3:6]
        xyz = origin[:, None, :] + dirs[:, None, :] * z_all[..., None]
        cam = data[..., 6:7].expand(-1, z_all.shape[-1]) if data.shape[-1] > 6 else None
        return Samples(xyz=xyz, dirs=dirs[:, None, :].expand_as(xyz), z_vals=z_all, camera_idx=cam,
                       rank=getattr(rays, "rank", None), group=getattr(rays, "group", None))

"""Losses and image metrics (reference: landmark/nerf_components/utils/loss_utils.py:14-265).

``eff_distloss`` is an O(N) prefix-sum evaluation of the mip-NeRF-360 distortion loss; the
reference imports it from the external ``torch_efficient_distloss`` package
(benchmarks/nerf/gridnerf/gridnerf.py:10,455-466).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn


def l1_loss(network_output: torch.Tensor, gt: torch.Tensor) -> torch.Tensor:
    return (network_output - gt).abs().mean()


def l2_loss(network_output: torch.Tensor, gt: torch.Tensor) -> torch.Tensor:
    return ((network_output - gt) ** 2).mean()


def _gaussian_window(size: int, sigma: float, channels: int, like: torch.Tensor) -> torch.Tensor:
    x = torch.arange(size, dtype=torch.float32) - size // 2
    g = torch.exp(-(x ** 2) / (2 * sigma ** 2))
    g = g / g.sum()
    w2d = g[:, None] @ g[None, :]
    return w2d.expand(channels, 1, size, size).contiguous().to(device=like.device, dtype=like.dtype)


def gaussian(window_size: int, sigma: float) -> torch.Tensor:
    """Normalised 1-D Gaussian of ``window_size`` taps centred on the middle tap."""
    x = torch.arange(window_size, dtype=torch.float32) - window_size // 2
    g = torch.exp(-(x ** 2) / (2 * sigma ** 2))
    return g / g.sum()


def create_window(window_size: int, channel: int) -> torch.Tensor:
    """Depth-wise SSIM filter ``[channel, 1, window_size, window_size]`` (sigma 1.5)."""
    return _gaussian_window(window_size, 1.5, channel, torch.zeros(()))


def ssim(img1: torch.Tensor, img2: torch.Tensor, window_size: int = 11, size_average: bool = True) -> torch.Tensor:
    """SSIM with an 11x11 Gaussian window (sigma 1.5); images are ``[C, H, W]`` or ``[N, C, H, W]``."""
    if img1.dim() == 3:
        img1, img2 = img1[None], img2[None]
    if img1.is_cuda:
        from ...ops.ssim import fused_ssim_available, fused_ssim

        if fused_ssim_available() and window_size == 11 and size_average:
            return fused_ssim(img1, img2)
    C = img1.shape[1]
    win = _gaussian_window(window_size, 1.5, C, img1)
    pad = window_size // 2
    mu1, mu2 = F.conv2d(img1, win, padding=pad, groups=C), F.conv2d(img2, win, padding=pad, groups=C)
    mu1_sq, mu2_sq, mu12 = mu1 * mu1, mu2 * mu2, mu1 * mu2
    s1 = F.conv2d(img1 * img1, win, padding=pad, groups=C) - mu1_sq
    s2 = F.conv2d(img2 * img2, win, padding=pad, groups=C) - mu2_sq
    s12 = F.conv2d(img1 * img2, win, padding=pad, groups=C) - mu12
    C1, C2 = 0.01 ** 2, 0.03 ** 2
    ssim_map = ((2 * mu12 + C1) * (2 * s12 + C2)) / ((mu1_sq + mu2_sq + C1) * (s1 + s2 + C2))
    return ssim_map.mean() if size_average else ssim_map.mean(dim=(1, 2, 3))


class TVLoss(nn.Module):
    """Total variation of ``[N, C, H, W]`` maps, normalised per element."""

    def __init__(self, TVLoss_weight: float = 1.0):
        super().__init__()
        self.TVLoss_weight = TVLoss_weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n, c, h, w = x.shape
        count_h, count_w = c * (h - 1) * w, c * h * (w - 1)
        h_tv = (x[:, :, 1:, :] - x[:, :, :-1, :]).pow(2).sum()
        w_tv = (x[:, :, :, 1:] - x[:, :, :, :-1]).pow(2).sum()
        return self.TVLoss_weight * 2 * (h_tv / count_h + w_tv / count_w) / n


# -- mip-NeRF-360 style losses --------------------------------------------------------------
def eff_distloss(w: torch.Tensor, m: torch.Tensor, interval: torch.Tensor) -> torch.Tensor:
    """Distortion loss  sum_ij w_i w_j |m_i - m_j| + 1/3 sum_i w_i^2 d_i  (mean over rays), computed
    with prefix sums assuming ``m`` is sorted along the last dim.  On CUDA one warp-per-ray kernel returns the loss
    and its gradient (``ops/csrc/ray_losses.cu``)."""
    if w.dim() == 2 and not (m.requires_grad or interval.requires_grad):
        from ...ops import ray_losses

        if ray_losses.kernels_usable(w, m, interval):
            return ray_losses.distortion_per_ray(w, m, interval).mean()
    loss_uni = (1.0 / 3.0) * (interval * w.pow(2)).sum(dim=-1).mean()
    wm = w * m
    w_cum, wm_cum = w.cumsum(-1), wm.cumsum(-1)
    loss_bi = 2.0 * (wm[..., 1:] * w_cum[..., :-1] - w[..., 1:] * wm_cum[..., :-1]).sum(dim=-1).mean()
    return loss_bi + loss_uni


def ray_samples_to_sdist(spacing_starts: torch.Tensor, spacing_ends: torch.Tensor) -> torch.Tensor:
    return torch.cat((spacing_starts[..., 0], spacing_ends[..., -1:, 0]), dim=-1)


def lossfun_distortion(t: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    ut = (t[..., 1:] + t[..., :-1]) / 2
    dut = (ut[..., :, None] - ut[..., None, :]).abs()
    inter = (w * (w[..., None, :] * dut).sum(-1)).sum(-1)
    intra = (w ** 2 * (t[..., 1:] - t[..., :-1])).sum(-1) / 3
    return inter + intra


def distortion_loss(weights_list, spacing_starts_list, spacing_ends_list) -> torch.Tensor:
    c = ray_samples_to_sdist(spacing_starts_list[-1], spacing_ends_list[-1])
    w = weights_list[-1][..., 0]
    if w.dim() == 2 and not c.requires_grad:
        from ...ops import ray_losses

        if ray_losses.kernels_usable(w, c):      # O(S) prefix sums in one kernel instead of the S x S matrix per ray
            return ray_losses.distortion_per_ray(w, (c[..., 1:] + c[..., :-1]) / 2, c[..., 1:] - c[..., :-1]).mean()
    return lossfun_distortion(c, w).mean()


def outer(t0_starts, t0_ends, t1_starts, t1_ends, y1):
    cy1 = torch.cat((torch.zeros_like(y1[..., :1]), torch.cumsum(y1, dim=-1)), dim=-1)
    lo = (torch.searchsorted(t1_starts.contiguous(), t0_starts.contiguous(), side="right") - 1).clamp(0, y1.shape[-1] - 1)
    hi = torch.searchsorted(t1_ends.contiguous(), t0_ends.contiguous(), side="right").clamp(0, y1.shape[-1] - 1)
    return torch.take_along_dim(cy1[..., 1:], hi, dim=-1) - torch.take_along_dim(cy1[..., :-1], lo, dim=-1)


def lossfun_outer(t, w, t_env, w_env):
    w_outer = outer(t[..., :-1], t[..., 1:], t_env[..., :-1], t_env[..., 1:], w_env)
    return torch.clip(w - w_outer, min=0) ** 2 / (w + 1e-7)


def interlevel_loss(weights_list, spacing_starts_list, spacing_ends_list) -> torch.Tensor:
    c = ray_samples_to_sdist(spacing_starts_list[-1], spacing_ends_list[-1]).detach()
    w = weights_list[-1][..., 0].detach()
    total = 0.0
    for weights, starts, ends in zip(weights_list[:-1], spacing_starts_list[:-1], spacing_ends_list[:-1]):
        t_env, w_env = ray_samples_to_sdist(starts, ends), weights[..., 0]
        if w.dim() == 2 and w_env.shape[-1] <= 1024 and not t_env.requires_grad:
            from ...ops import ray_losses

            if ray_losses.kernels_usable(w, w_env, c, t_env):
                total = total + ray_losses.interlevel_per_ray(c, w, t_env, w_env).sum() / w.numel()
                continue
        total = total + lossfun_outer(c, w, t_env, w_env).mean()
    return total


# -- numpy metrics ------------------------------------------------------------------------
_LPIPS = {}


def init_lpips(net_name: str, device):
    """The LPIPS network ``"alex"`` / ``"vgg"`` on ``device``, or ``None`` when the external ``lpips`` package (and
    its pretrained weights) is not installed."""
    assert net_name in ("alex", "vgg")
    try:
        import lpips
    except ImportError:
        return None
    return lpips.LPIPS(net=net_name, version="0.1").eval().to(device)


def rgb_lpips(np_gt, np_im, net_name: str, device):
    """LPIPS needs the external ``lpips`` package and its pretrained weights; ``nan`` without them."""
    if net_name not in _LPIPS:
        _LPIPS[net_name] = init_lpips(net_name, device)
    if _LPIPS[net_name] is None:
        return float("nan")
    gt = torch.from_numpy(np_gt).permute(2, 0, 1).contiguous().to(device)
    im = torch.from_numpy(np_im).permute(2, 0, 1).contiguous().to(device)
    return _LPIPS[net_name](gt, im, normalize=True).item()


def rgb_ssim(img0, img1, max_val, filter_size=11, filter_sigma=1.5, k1=0.01, k2=0.03, return_map=False):
    """SSIM on ``[H, W, 3]`` numpy images with a separable Gaussian, valid region only."""
    from scipy.signal import convolve2d

    hw = filter_size // 2
    f = np.exp(-0.5 * ((np.arange(filter_size) - hw + (1 - filter_size % 2) / 2) / filter_sigma) ** 2)
    f /= f.sum()

    def blur(z):
        return np.stack([convolve2d(convolve2d(z[..., i], f[:, None], mode="valid"), f[None, :], mode="valid")
                         for i in range(z.shape[-1])], -1)

    mu0, mu1 = blur(img0), blur(img1)
    s00 = np.maximum(0.0, blur(img0 ** 2) - mu0 * mu0)
    s11 = np.maximum(0.0, blur(img1 ** 2) - mu1 * mu1)
    s01 = blur(img0 * img1) - mu0 * mu1
    s01 = np.sign(s01) * np.minimum(np.sqrt(s00 * s11), np.abs(s01))
    c1, c2 = (k1 * max_val) ** 2, (k2 * max_val) ** 2
    ssim_map = ((2 * mu0 * mu1 + c1) * (2 * s01 + c2)) / ((mu0 ** 2 + mu1 ** 2 + c1) * (s00 + s11 + c2))
    return ssim_map if return_map else float(ssim_map.mean())

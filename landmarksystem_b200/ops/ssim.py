"""Fused L1 + SSIM image loss (``csrc/ssim.cu``): one kernel forward, one backward, for ``[C, H, W]`` or
``[N, C, H, W]`` fp32 images.  ``fused_l1_ssim`` returns ``(l1_mean, ssim_mean)`` so that callers can weight
them (3DGS: ``(1 - lambda) * l1 + lambda * (1 - ssim)``); ``fused_ssim`` returns the SSIM mean alone."""
from __future__ import annotations

from ctypes import c_int

import torch

from . import native

P = native.P
native.register_signature("lmb_ssim_fwd", [P, P, c_int, c_int, c_int, P, P, P, P, P])
native.register_signature("lmb_ssim_bwd", [P, P, P, P, P, c_int, c_int, c_int, P, P, P])


def fused_ssim_available() -> bool:
    return native.available()


class _L1SSIM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, img, gt):
        x = img.contiguous().float()
        y = gt.contiguous().float()
        H, W = x.shape[-2:]
        C = x.numel() // (H * W)
        sums = torch.zeros(2, device=x.device, dtype=torch.float32)
        need = img.requires_grad
        maps = torch.empty((3,) + tuple(x.shape), device=x.device, dtype=torch.float32) if need else None
        native.check(native.lib().lmb_ssim_fwd(x.data_ptr(), y.data_ptr(), C, H, W, sums.data_ptr(),
                                               native.ptr(maps[0] if need else None), native.ptr(maps[1] if need else None),
                                               native.ptr(maps[2] if need else None), native.stream_ptr()), "ssim_fwd")
        ctx.save_for_backward(x, y, maps)
        ctx.dims = (C, H, W)
        means = sums / float(x.numel())
        return means[0], means[1]

    @staticmethod
    def backward(ctx, d_l1, d_ssim):
        x, y, maps = ctx.saved_tensors
        C, H, W = ctx.dims
        n = float(x.numel())
        zero = torch.zeros((), device=x.device)
        scales = torch.stack(((d_l1 if d_l1 is not None else zero) / n, (d_ssim if d_ssim is not None else zero) / n)).float()
        dx = torch.empty_like(x)
        native.check(native.lib().lmb_ssim_bwd(x.data_ptr(), y.data_ptr(), maps[0].data_ptr(), maps[1].data_ptr(),
                                               maps[2].data_ptr(), C, H, W, scales.contiguous().data_ptr(), dx.data_ptr(),
                                               native.stream_ptr()), "ssim_bwd")
        return dx, None


def fused_l1_ssim(img: torch.Tensor, gt: torch.Tensor):
    """``(mean |img - gt|, mean SSIM)``; gradients flow to ``img``."""
    return _L1SSIM.apply(img, gt)


def fused_ssim(img1: torch.Tensor, img2: torch.Tensor) -> torch.Tensor:
    return _L1SSIM.apply(img1, img2)[1]

"""Volume-rendering composite ops (weights scan and weighted colour/depth sums).

CPU tensors run the PyTorch statement of the math (the oracle); CUDA tensors run the warp-scan
kernels in ``csrc/composite.cu``.  Reference behaviour:
landmark/nerf_components/model_components/renderers/volume_renderer.py:20-67.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import native


def weights_reference(sigma: torch.Tensor, dists: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    alpha = 1.0 - torch.exp(-sigma * dists)
    trans = torch.cumprod(torch.cat([torch.ones_like(alpha[:, :1]), 1.0 - alpha + 1e-10], -1), -1)
    return alpha * trans[:, :-1], trans[:, -1]


def render_reference(weights, rgbs, z_vals, bg: float):
    acc = weights.sum(-1)
    rgb = (weights[..., None] * rgbs).sum(-2) + bg * (1.0 - acc[..., None])
    depth = (weights * z_vals).sum(-1)
    return rgb, depth, acc


class _Weights(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sigma, dists):
        R, S = sigma.shape
        weights = torch.empty_like(sigma)
        bg = torch.empty(R, device=sigma.device, dtype=torch.float32)
        native.check(native.lib().lmb_weights_fwd(sigma.data_ptr(), dists.data_ptr(), R, S, weights.data_ptr(),
                                                  bg.data_ptr(), native.stream_ptr()), "weights_fwd")
        ctx.save_for_backward(sigma, dists)
        return weights, bg

    @staticmethod
    def backward(ctx, dweights, dbg):
        sigma, dists = ctx.saved_tensors
        R, S = sigma.shape
        dsigma = torch.empty_like(sigma)
        dweights = dweights.contiguous()
        dbg = None if dbg is None else dbg.contiguous()
        native.check(native.lib().lmb_weights_bwd(sigma.data_ptr(), dists.data_ptr(), dweights.data_ptr(),
                                                  native.ptr(dbg), R, S, dsigma.data_ptr(), native.stream_ptr()),
                     "weights_bwd")
        return dsigma, None


class _Render(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weights, rgbs, z_vals, bg):
        R, S = weights.shape
        rgb = torch.empty((R, 3), device=weights.device, dtype=torch.float32)
        depth = torch.empty(R, device=weights.device, dtype=torch.float32)
        acc = torch.empty(R, device=weights.device, dtype=torch.float32)
        native.check(native.lib().lmb_render_fwd(weights.data_ptr(), rgbs.data_ptr(), z_vals.data_ptr(), R, S,
                                                 float(bg), rgb.data_ptr(), depth.data_ptr(), acc.data_ptr(),
                                                 native.stream_ptr()), "render_fwd")
        ctx.save_for_backward(weights, rgbs)
        ctx.bg = float(bg)
        ctx.mark_non_differentiable(depth, acc)
        return rgb, depth, acc

    @staticmethod
    def backward(ctx, drgb, _ddepth, _dacc):
        weights, rgbs = ctx.saved_tensors
        R, S = weights.shape
        dweights = torch.empty_like(weights)
        drgbs = torch.empty_like(rgbs)
        drgb = drgb.contiguous()
        native.check(native.lib().lmb_render_bwd(weights.data_ptr(), rgbs.data_ptr(), drgb.data_ptr(), R, S, ctx.bg,
                                                 dweights.data_ptr(), drgbs.data_ptr(), native.stream_ptr()),
                     "render_bwd")
        return dweights, drgbs, None, None


def composite_weights(sigma: torch.Tensor, dists: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(weights [R,S], bg_transmittance [R])`` from densities and inter-sample distances."""
    if not sigma.is_cuda:
        return weights_reference(sigma, dists)
    return _Weights.apply(sigma.contiguous().float(), dists.contiguous().float())


def composite_render(weights: torch.Tensor, rgbs: torch.Tensor, z_vals: torch.Tensor, bg: float = 0.0):
    """``(rgb [R,3] unclamped, depth [R], acc [R])``; depth/acc carry no gradient (as in the reference)."""
    if not weights.is_cuda:
        rgb, depth, acc = render_reference(weights, rgbs, z_vals, bg)
        return rgb, depth.detach(), acc.detach()
    return _Render.apply(weights.contiguous().float(), rgbs.contiguous().float(), z_vals.contiguous().float(), bg)

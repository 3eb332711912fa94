"""Volume renderer: weights from densities, then colour/depth composite (reference:
landmark/nerf_components/model_components/renderers/volume_renderer.py:6-67).  The math runs in
the warp-scan CUDA kernels on GPU tensors and in PyTorch on CPU tensors."""
from __future__ import annotations

import torch

from ...ops import composite_render, composite_weights
from .base_renderer import BaseRenderer


class VolumeRenderer(BaseRenderer):
    def __init__(self, white_bg: bool = False) -> None:
        super().__init__()
        self.white_bg = white_bg
        self.save_init_kwargs(locals())

    def get_weights(self, sigma: torch.Tensor, distances: torch.Tensor) -> torch.Tensor:
        return composite_weights(sigma, distances)[0]

    def forward(self, weights: torch.Tensor, rgbs: torch.Tensor, z_vals: torch.Tensor,
                random_white_bg_ratio: float = 0.0):
        if not self.white_bg and random_white_bg_ratio > 0.0 and weights.is_cuda:
            # the coin is tossed on the device: no host decision is baked in when the step is recorded in a CUDA graph
            bg = (torch.rand((), device=weights.device) < random_white_bg_ratio).to(weights.dtype)
            rgb_map, depth_map, _ = composite_render(weights, rgbs, z_vals, 0.0)
            rgb_map = rgb_map + bg * (1.0 - weights.sum(-1, keepdim=True))
            return rgb_map.clamp(0, 1), depth_map
        white = self.white_bg or (random_white_bg_ratio > 0.0 and float(torch.rand(())) < random_white_bg_ratio)
        rgb_map, depth_map, _ = composite_render(weights, rgbs, z_vals, 1.0 if white else 0.0)
        return rgb_map.clamp(0, 1), depth_map


class FusedVolumeRenderer(VolumeRenderer):
    """Kernel-runtime name; the reference's class is an empty stub
    (model_components/renderers/fused_volume_renderer.py)."""

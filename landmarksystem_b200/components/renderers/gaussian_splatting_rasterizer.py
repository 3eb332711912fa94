"""Renderer component for explicit 3D Gaussians (reference: the interface stub
landmark/nerf_components/model_components/renderers/gaussian_splatting_rasterizer.py:4-13, whose ``forward`` takes a
list of models and is left empty there).

``forward(model, camera)`` rasterises the Gaussians of one model, or of several models at once: the primitives of every
model in the list are concatenated and sorted together by the rasteriser, so scene parts trained as separate models
(spatial blocks) blend in correct depth order - which compositing their separately rendered images cannot give.
"""
from __future__ import annotations

import math
from typing import Dict, Sequence, Union

import torch

from ...ops.gaussian_raster import GaussianRasterizationSettings, GaussianRasterizer
from .base_renderer import BaseRenderer


def _encoding_of(model):
    return getattr(model, "gaussian_encoding", model)


class GaussianSplattingRasterizer(BaseRenderer):
    def __init__(self, white_background: bool = False, debug: bool = False):
        super().__init__()
        self.white_background, self.debug = white_background, debug
        self.rasterizer = GaussianRasterizer(None)

    def settings_for(self, camera, sh_degree: int, device, scaling_modifier: float = 1.0, background=None):
        bg = background if background is not None else torch.full((3,), 1.0 if self.white_background else 0.0, device=device)
        return GaussianRasterizationSettings(
            image_height=int(camera.image_height), image_width=int(camera.image_width),
            tanfovx=math.tan(camera.FoVx * 0.5), tanfovy=math.tan(camera.FoVy * 0.5), bg=bg.to(device),
            scale_modifier=scaling_modifier, viewmatrix=camera.world_view_transform,
            projmatrix=camera.full_proj_transform, sh_degree=sh_degree, campos=camera.camera_center,
            prefiltered=False, debug=self.debug)

    def forward(self, model: Union[object, Sequence[object]], camera=None, scaling_modifier: float = 1.0,
                background=None, **kwargs) -> Dict[str, torch.Tensor]:
        """``model``: a Gaussian model / encoding or a list of them (same SH degree).  Returns ``render [3, H, W]``,
        ``radii [N]``, ``visibility_filter [N]``, ``viewspace_points [N, 3]`` (gradient carrier of the screen-space
        means) and ``counts`` (primitives per model, in list order, to split the per-primitive outputs)."""
        assert camera is not None, "a camera is required"
        encodings = [_encoding_of(m) for m in (model if isinstance(model, (list, tuple)) else [model])]
        assert encodings, "nothing to render"
        device = encodings[0].get_xyz.device
        camera = camera.to(device)
        degrees = {int(e.active_sh_degree) for e in encodings}
        widths = {int(e.get_features.shape[1]) for e in encodings}
        assert len(widths) == 1, "the models must carry the same number of SH coefficients"
        cat = (lambda name: getattr(encodings[0], name)) if len(encodings) == 1 else \
            (lambda name: torch.cat([getattr(e, name) for e in encodings], dim=0))
        means3D, opacity, scales, rotations, shs = (cat(n) for n in
                                                    ("get_xyz", "get_opacity", "get_scaling", "get_rotation", "get_features"))
        screenspace = torch.zeros_like(means3D, requires_grad=True) + 0
        if screenspace.requires_grad:
            screenspace.retain_grad()
        self.rasterizer.raster_settings = self.settings_for(camera, min(degrees), device, scaling_modifier, background)
        image, radii, _ = self.rasterizer(means3D=means3D, means2D=screenspace, shs=shs, colors_precomp=None,
                                          opacities=opacity, scales=scales, rotations=rotations, cov3D_precomp=None)
        return {"render": image, "radii": radii, "visibility_filter": radii > 0, "viewspace_points": screenspace,
                "counts": [int(e.get_xyz.shape[0]) for e in encodings]}


GassianSplattingRasterizer = GaussianSplattingRasterizer          # the reference's spelling of the class name

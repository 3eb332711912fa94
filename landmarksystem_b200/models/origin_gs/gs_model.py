"""Vanilla 3D Gaussian splatting model (reference: benchmarks/nerf/origin_gs/gs_model.py:15-339)."""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ...components.fields.encodings.gaussian_encoding import GaussianEncoding
from ...components.model.base_model import BaseGaussian
from ...components.utils.sh_utils import eval_sh
from ...configs import ConfigClass
from ...ops.gaussian_raster import GaussianRasterizationSettings, GaussianRasterizer


class Gaussian3DConfig(ConfigClass):
    sh_degree: int = 3
    images: str = "images"
    model_path: Optional[str] = None
    position_lr_init: float = 0.00016
    position_lr_final: float = 0.0000016
    position_lr_delay_mult: float = 0.01
    position_lr_max_steps: int = 30000
    feature_lr: float = 0.0025
    opacity_lr: float = 0.05
    scaling_lr: float = 0.005
    rotation_lr: float = 0.001
    percent_dense: float = 0.01
    lambda_dssim: float = 0.2
    densification_interval: int = 100
    opacity_reset_interval: int = 3000
    densify_from_iter: int = 500
    densify_until_iter: int = 15000
    densify_grad_threshold: float = 0.0002
    convert_SHs_python: bool = False
    compute_cov3D_python: bool = False
    no_batching: bool = False
    white_bkgd: bool = False
    resolution: int = -1
    resolution_scales: List[float] = [1.0]
    point_path: Optional[str] = None
    max_init_points: int = -1
    neighbour_size: int = 1
    init_points_num: int = 100000
    init_points_volume: bool = False   # draw the random initial cloud inside the AABB instead of on its floor
    act_cache: bool = False


def raster_settings_for(camera, background, sh_degree: int, scaling_modifier: float = 1.0, debug: bool = False):
    return GaussianRasterizationSettings(
        image_height=int(camera.image_height), image_width=int(camera.image_width),
        tanfovx=math.tan(camera.FoVx * 0.5), tanfovy=math.tan(camera.FoVy * 0.5), bg=background,
        scale_modifier=scaling_modifier, viewmatrix=camera.world_view_transform,
        projmatrix=camera.full_proj_transform, sh_degree=sh_degree, campos=camera.camera_center,
        prefiltered=False, debug=debug)


class GaussianModel(BaseGaussian):
    def __init__(self, config, scene_manager=None, cam_extent=None):
        super().__init__(config, scene_manager)
        self.cam_extent = cam_extent
        dev = config.device if torch.cuda.is_available() or str(config.device) == "cpu" else "cpu"
        self.device = torch.device(dev)
        self.background = torch.tensor([1.0, 1, 1] if config.white_bkgd else [0.0, 0, 0], device=self.device)
        self.spatial_lr_scale = 0
        self.init_field_components()
        self.init_renderer()

    def init_field_components(self):
        cfg = self.config
        self.gaussian_encoding = GaussianEncoding(sh_degree=cfg.sh_degree, percent_dense=cfg.percent_dense,
                                                  act_cache=cfg.act_cache, device=self.device)

    def init_renderer(self):
        self.renderer = GaussianRasterizer(None)

    def construct_list_of_attributes(self):
        return self.gaussian_encoding.construct_list_of_attributes()

    def construct_list_of_cache_attributes(self):
        return self.gaussian_encoding.construct_list_of_cache_attributes()

    def create_from_pcd(self, pcd, spatial_lr_scale: float):
        self.spatial_lr_scale = spatial_lr_scale
        self.gaussian_encoding.create_from_pcd(pcd)

    def oneupSHdegree(self):
        self.gaussian_encoding.oneupSHdegree()

    def train(self, mode: bool = True):
        self.gaussian_encoding.clear_cache()
        return super().train(mode)

    # -- rendering ----------------------------------------------------------------------------------
    def prefilter_voxel(self, camera, scaling_modifier: float = 1.0) -> torch.Tensor:
        """Boolean visibility of every Gaussian for this view (frustum + extent test, no rendering)."""
        enc, cfg = self.gaussian_encoding, self.config
        rast = GaussianRasterizer(raster_settings_for(camera, self.background, 1, scaling_modifier, cfg.debug))
        if cfg.compute_cov3D_python:
            radii = rast.visible_filter(enc.get_xyz, cov3D_precomp=enc.get_covariance(scaling_modifier))
        else:
            radii = rast.visible_filter(enc.get_xyz, scales=enc.get_scaling[:, :3], rotations=enc.get_rotation)
        return radii > 0

    def forward(self, viewpoint_camera, scaling_modifier: float = 1.0, override_color=None, render_exclude_filter=None):
        enc, cfg = self.gaussian_encoding, self.config
        cam = viewpoint_camera.to(self.device)
        if self.training or render_exclude_filter is not None or not enc.get_xyz.is_cuda:
            visible = self.prefilter_voxel(cam, scaling_modifier)
            if render_exclude_filter is not None:
                visible = visible & render_exclude_filter
        else:
            visible = None       # evaluation on the GPU: the rasteriser's own preprocess kernel does the same frustum test
        means3D = enc.get_xyz
        screenspace = torch.zeros_like(means3D, requires_grad=True) + 0
        if self.training:
            screenspace.retain_grad()
        self.renderer.raster_settings = raster_settings_for(cam, self.background, enc.active_sh_degree,
                                                            scaling_modifier, cfg.debug)
        opacity = enc.get_opacity
        scales = rotations = cov3D = shs = colors = None
        if cfg.compute_cov3D_python:
            cov3D = enc.get_covariance(scaling_modifier)
        else:
            scales, rotations = enc.get_scaling, enc.get_rotation
        if override_color is not None:
            colors = override_color
        elif cfg.convert_SHs_python:
            feats = enc.get_features.transpose(1, 2)
            dirs = means3D - cam.camera_center[None]
            dirs = dirs / dirs.norm(dim=1, keepdim=True)
            colors = torch.clamp_min(eval_sh(enc.active_sh_degree, feats, dirs) + 0.5, 0.0)
        else:
            shs = enc.get_features
        means2D = screenspace
        # The reference compacts every per-Gaussian tensor to the visible subset before an evaluation render
        # (benchmarks/nerf/origin_gs/gs_model.py:199-208) because its rasteriser preprocesses whatever it is given; the
        # rasteriser here takes the visibility mask and skips masked Gaussians in its first kernel, so no index list is
        # built on the host and no gigabyte of parameters is gathered per frame.
        mask = visible
        image, radii, _ = self.renderer(means3D=means3D, means2D=means2D, shs=shs, colors_precomp=colors,
                                        opacities=opacity, scales=scales, rotations=rotations, cov3D_precomp=cov3D,
                                        visible_mask=mask)
        self.viewspace_points, self.visibility_filter, self.radii = screenspace, (visible if visible is not None else radii > 0), radii
        return image

    # -- training helpers -------------------------------------------------------------------------------
    def densification(self, optimizer, iteration: int):
        cfg, enc = self.config, self.gaussian_encoding
        if iteration >= cfg.densify_until_iter:
            return
        vis = self.visibility_filter
        enc.max_radii2D[vis] = torch.max(enc.max_radii2D[vis], self.radii[vis].float())
        enc.add_densification_stats(self.viewspace_points, vis)
        if iteration > cfg.densify_from_iter and iteration % cfg.densification_interval == 0:
            size_threshold = 20 if iteration > cfg.opacity_reset_interval else None
            enc.densify_and_prune(cfg.densify_grad_threshold, 0.005, self.cam_extent, size_threshold, optimizer)
        if iteration % cfg.opacity_reset_interval == 0 or (cfg.white_bkgd and iteration == cfg.densify_from_iter):
            enc.reset_opacity(optimizer)

    def get_optparam_groups(self, training_args):
        e, a = self.gaussian_encoding, training_args
        return [
            {"params": [e._xyz], "lr": a.position_lr_init * self.spatial_lr_scale, "name": "xyz"},
            {"params": [e._features_dc], "lr": a.feature_lr, "name": "f_dc"},
            {"params": [e._features_rest], "lr": a.feature_lr / 20.0, "name": "f_rest"},
            {"params": [e._opacity], "lr": a.opacity_lr, "name": "opacity"},
            {"params": [e._scaling], "lr": a.scaling_lr, "name": "scaling"},
            {"params": [e._rotation], "lr": a.rotation_lr, "name": "rotation"},
        ]

    @property
    def get_primitives_num(self) -> int:
        return len(self.gaussian_encoding._xyz)

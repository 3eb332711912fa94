"""Scaffold-GS: anchors + neural Gaussians decoded per view (reference:
benchmarks/nerf/scaffold_gs/gs_model.py:18-444)."""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from ...components.fields.anchor_decoder import AnchorDecoder
from ...components.fields.encodings.scaffoldgs_encoding import ScaffoldGSEncoding
from ...components.model.base_model import BaseGaussian
from ...configs import ConfigClass
from ...ops.gaussian_raster import GaussianRasterizer
from ..origin_gs.gs_model import raster_settings_for


class ScaffoldGSConfig(ConfigClass):
    sh_degree: int = 3
    images: str = "images"
    model_path: Optional[str] = None
    source_path: Optional[str] = None
    feat_dim: int = 32
    view_dim: int = 3
    n_offsets: int = 10
    voxel_size: float = 0.001
    update_depth: int = 3
    update_init_factor: int = 16
    update_hierachy_factor: int = 4
    use_feat_bank: bool = False
    add_opacity_dist: bool = True
    add_cov_dist: bool = True
    add_color_dist: bool = True
    add_level: bool = False
    appearance_dim: int = 0
    lod: int = 0
    feature_lr: float = 0.0075
    opacity_lr: float = 0.02
    scaling_lr: float = 0.007
    rotation_lr: float = 0.002
    position_lr_init: float = 0.0
    position_lr_final: float = 0.0
    position_lr_delay_mult: float = 0.01
    position_lr_max_steps: int = 30000
    offset_lr_init: float = 0.01
    offset_lr_final: float = 0.0001
    offset_lr_delay_mult: float = 0.01
    offset_lr_max_steps: int = 30000
    mlp_opacity_lr_init: float = 0.002
    mlp_opacity_lr_final: float = 0.00002
    mlp_opacity_lr_delay_mult: float = 0.01
    mlp_opacity_lr_max_steps: int = 30000
    mlp_cov_lr_init: float = 0.004
    mlp_cov_lr_final: float = 0.004
    mlp_cov_lr_delay_mult: float = 0.01
    mlp_cov_lr_max_steps: int = 30000
    mlp_color_lr_init: float = 0.008
    mlp_color_lr_final: float = 0.00005
    mlp_color_lr_delay_mult: float = 0.01
    mlp_color_lr_max_steps: int = 30000
    mlp_featurebank_lr_init: float = 0.01
    mlp_featurebank_lr_final: float = 0.00001
    mlp_featurebank_lr_delay_mult: float = 0.01
    mlp_featurebank_lr_max_steps: int = 30000
    appearance_lr_init: float = 0.05
    appearance_lr_final: float = 0.0005
    appearance_lr_delay_mult: float = 0.01
    appearance_lr_max_steps: int = 30000
    percent_dense: float = 0.01
    lambda_dssim: float = 0.2
    start_stat: int = 500
    update_from: int = 1500
    update_interval: int = 100
    update_until: int = 15000
    min_opacity: float = 0.005
    success_threshold: float = 0.8
    densify_grad_threshold: float = 0.0002
    no_batching: bool = False
    white_bkgd: bool = False
    resolution: float = -1
    resolution_scales: List[float] = [1.0]
    point_path: Optional[str] = None
    max_init_points: int = -1
    neighbour_size: int = 1
    init_points_num: int = 100000
    init_points_volume: bool = False
    runtime: str = "Torch"
    kernel_fusion: bool = False
    # accepted from the reference's configuration files (scaffold_gs/gs_model.py:86-87, octree_gs/gs_model.py:33-41)
    convert_SHs_python: bool = False            # no effect: colours come from the anchor decoder
    compute_cov3D_python: bool = False          # pre-filter anchors with covariances built in PyTorch
    white_background: bool = False
    random_background: bool = False
    data_device: str = "cuda"
    eval: bool = False
    ds: int = 1
    ratio: int = 1                              # keep every ``ratio``-th input point (Octree-GS initialisation)
    undistorted: bool = False


class ScaffoldGS(BaseGaussian):
    """Shared by Octree-GS (which overrides the encoding, the per-view mask and the decoder inputs)."""

    def __init__(self, config, scene_manager=None, cam_extent=None):
        super().__init__(config, scene_manager)
        self.cam_extent = cam_extent
        dev = config.device if torch.cuda.is_available() or str(config.device) == "cpu" else "cpu"
        self.device = torch.device(dev)
        self.background = torch.tensor([1.0, 1, 1] if config.white_bkgd else [0.0, 0, 0], device=self.device)
        self.spatial_lr_scale = 0
        self.use_feat_bank = config.use_feat_bank
        self.init_field_components()
        self.init_renderer()

    # -- construction ----------------------------------------------------------------------------------
    def init_field_components(self):
        c = self.config
        self.gaussian_encoding = ScaffoldGSEncoding(c.feat_dim, c.n_offsets, c.voxel_size, c.update_depth,
                                                    c.update_init_factor, c.update_hierachy_factor, c.percent_dense,
                                                    device=self.device)
        self._init_decoder()

    def _init_decoder(self, dist2level=None):
        c = self.config
        self.anchor_decoder = AnchorDecoder(c.use_feat_bank, c.add_opacity_dist, c.add_color_dist, c.add_cov_dist,
                                            c.view_dim, c.feat_dim, c.n_offsets, appearance_dim=c.appearance_dim,
                                            add_level=c.add_level, dist2level=dist2level).to(self.device)
        if c.get("runtime", "Torch") == "Kernel" or c.get("kernel_fusion", False):
            self.anchor_decoder.use_fused = True
        self.embedding_appearance = None

    def set_appearance(self, num_cameras: int):
        if self.config.appearance_dim > 0:
            self.embedding_appearance = torch.nn.Embedding(num_cameras, self.config.appearance_dim).to(self.device)

    def get_appearance_code(self, appearance_code_idx):
        return self.embedding_appearance(appearance_code_idx)

    def save_mlp_checkpoints(self, path: str):
        """The decoder heads (and feature bank / appearance embedding when present) in one file with the reference's
        keys (scaffold_gs/gs_model.py, ``save_mlp_checkpoints``)."""
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        dec = self.anchor_decoder
        out = {"anchor_decoder.opacity_mlp": dec.mlp_opacity.state_dict(),
               "anchor_decoder.cov_mlp": dec.mlp_cov.state_dict(),
               "anchor_decoder.color_mlp": dec.mlp_color.state_dict()}
        if self.config.use_feat_bank and getattr(dec, "mlp_feature_bank", None) is not None:
            out["anchor_decoder.mlp_feature_bank"] = dec.mlp_feature_bank.state_dict()
        if self.embedding_appearance is not None:
            out["anchor_decoder.embedding_appearance"] = self.embedding_appearance.state_dict()
        torch.save(out, path)

    def init_renderer(self):
        self.renderer = GaussianRasterizer(None)

    def create_from_pcd(self, pcd, spatial_lr_scale: float):
        self.spatial_lr_scale = spatial_lr_scale
        self.gaussian_encoding.create_from_pcd(pcd)

    # -- rendering ------------------------------------------------------------------------------------------
    def prefilter_voxel(self, camera, anchor_mask=None, scaling_modifier: float = 1.0) -> torch.Tensor:
        enc = self.gaussian_encoding
        rast = GaussianRasterizer(raster_settings_for(camera, self.background, 1, scaling_modifier, self.config.debug))
        if self.config.get("compute_cov3D_python", False):
            cov = enc.get_covariance(1.0)       # the rasteriser settings already carry ``scaling_modifier``
            if anchor_mask is None:
                return rast.visible_filter(enc.get_anchor, cov3D_precomp=cov) > 0
            idx = anchor_mask.nonzero().squeeze(-1)
            radii = rast.visible_filter(enc.get_anchor[idx], cov3D_precomp=cov[idx])
            out = torch.zeros_like(anchor_mask)
            out[idx] = radii > 0
            return out
        if anchor_mask is None:
            radii = rast.visible_filter(enc.get_anchor, scales=enc.get_scaling[:, :3], rotations=enc.get_rotation)
            return radii > 0
        idx = anchor_mask.nonzero().squeeze(-1)
        radii = rast.visible_filter(enc.get_anchor[idx], scales=enc.get_scaling[idx, :3], rotations=enc.get_rotation[idx])
        out = torch.zeros_like(anchor_mask)
        out[idx] = radii > 0
        return out

    def _view_mask(self, cam):
        return self.prefilter_voxel(cam)

    def _decode(self, cam, visible):
        enc = self.gaussian_encoding
        app = None
        if self.embedding_appearance is not None:
            app = self.embedding_appearance(torch.tensor(self._appearance_index(cam), device=self.device))
        return self.anchor_decoder(cam.camera_center, enc.get_anchor, enc._anchor_feat, enc._offset, enc.get_scaling,
                                   visible, appearance_code=app)

    def _appearance_index(self, cam) -> int:
        """Row of the appearance embedding for this view: the camera's own while training or when no code was asked
        for, else the requested ``ape_code`` (reference: octree_gs/gs_model.py:254-260)."""
        code = int(getattr(self, "_ape_code", -1))
        return int(cam.uid) if (self.training or code < 0) else code

    def forward(self, viewpoint_camera, scaling_modifier: float = 1.0, retain_grad: bool = False,
                render_exclude_filter=None, ape_code: int = -1):
        """``render_exclude_filter``: optional ``[n_anchors]`` mask ANDed with the visibility of the anchors;
        ``ape_code``: appearance-embedding row to render with outside training (``-1``: the camera's own)."""
        cam = viewpoint_camera.to(self.device)
        self._ape_code = ape_code
        visible = self._view_mask(cam)
        if render_exclude_filter is not None:
            visible = visible & render_exclude_filter.to(visible.device)
        xyz, color, opacity, scaling, rot, neural_opacity, mask = self._decode(cam, visible)
        screenspace = torch.zeros_like(xyz, requires_grad=True) + 0
        if self.training:
            screenspace.retain_grad()
        self.renderer.raster_settings = raster_settings_for(cam, self.background, 1, scaling_modifier, self.config.debug)
        image, radii, _ = self.renderer(means3D=xyz, means2D=screenspace, shs=None, colors_precomp=color,
                                        opacities=opacity, scales=scaling, rotations=rot, cov3D_precomp=None)
        self.viewspace_points, self.visibility_filter, self.radii = screenspace, radii > 0, radii
        self.voxel_visible_mask, self.opacity, self.offset_selection_mask = visible, neural_opacity, mask
        self.scaling = scaling
        return image

    # -- training helpers ---------------------------------------------------------------------------------------
    def _adjust(self, optimizer, iteration):
        c = self.config
        self.gaussian_encoding.adjust_anchor(check_interval=c.update_interval, success_threshold=c.success_threshold,
                                             grad_threshold=c.densify_grad_threshold, min_opacity=c.min_opacity,
                                             optimizer=optimizer)

    def densification(self, optimizer, iteration: int):
        c, enc = self.config, self.gaussian_encoding
        if c.start_stat < iteration < c.update_until:
            enc.training_statis(self.viewspace_points, self.opacity, self.visibility_filter,
                                self.offset_selection_mask, self.voxel_visible_mask)
            if iteration > c.update_from and iteration % c.update_interval == 0:
                self._adjust(optimizer, iteration)

    def get_optparam_groups(self, a):
        e, d, s = self.gaussian_encoding, self.anchor_decoder, self.spatial_lr_scale
        groups = [
            {"params": [e._anchor], "lr": a.position_lr_init * s, "name": "anchor"},
            {"params": [e._offset], "lr": a.offset_lr_init * s, "name": "offset"},
            {"params": [e._anchor_feat], "lr": a.feature_lr, "name": "anchor_feat"},
            {"params": [e._opacity], "lr": a.opacity_lr, "name": "opacity"},
            {"params": [e._scaling], "lr": a.scaling_lr, "name": "scaling"},
            {"params": [e._rotation], "lr": a.rotation_lr, "name": "rotation"},
            {"params": list(d.mlp_opacity.parameters()), "lr": a.mlp_opacity_lr_init, "name": "mlp_opacity"},
            {"params": list(d.mlp_cov.parameters()), "lr": a.mlp_cov_lr_init, "name": "mlp_cov"},
            {"params": list(d.mlp_color.parameters()), "lr": a.mlp_color_lr_init, "name": "mlp_color"},
        ]
        if self.use_feat_bank:
            groups.append({"params": list(d.mlp_feature_bank.parameters()), "lr": a.mlp_featurebank_lr_init,
                           "name": "mlp_featurebank"})
        if self.embedding_appearance is not None:
            groups.append({"params": list(self.embedding_appearance.parameters()), "lr": a.appearance_lr_init,
                           "name": "embedding_appearance"})
        return groups

    @property
    def get_primitives_num(self) -> int:
        return len(self.gaussian_encoding._anchor)

"""Nerfacto: InstantNGP-style field with L-infinity scene contraction and proposal-network sampling
(reference: benchmarks/nerf/nerfacto/nerfacto.py:25-493)."""
from __future__ import annotations

from typing import List, Optional, Tuple, Union

import numpy as np
import torch
from torch import nn
from pydantic import model_validator
from typing_extensions import Literal

from ...components.data.rays import Rays
from ...components.fields.encodings.hash_encoding import HashEncoding
from ...components.fields.encodings.sh_encoding import SHEncoding
from ...components.fields.mlp_decoder import MLPDecoder
from ...components.model.base_model import BaseNeRF
from ...components.ray_samplers.proposal_network_sampler import ProposalNetworks, ProposalNetworkSampler
from ...components.renderers import VolumeRenderer
from ...components.utils.activation_utils import trunc_exp
from ...configs import ConfigClass
from ...ops import composite_render
from ..instant_ngp.instant_ngp import get_normalized_directions, window_block_ids


class NerfactoConfig(ConfigClass):
    num_levels: int = 16
    base_res: int = 16
    max_res: int = 2048
    log2_hashmap_size: int = 19
    features_per_level: int = 2
    hidden_dim: int = 64
    hidden_dim_color: int = 64
    appearance_embedding_dim: int = 32
    appearance_embed_dim: Optional[int] = None      # the reference's spelling (nerfacto.py:47); wins when given
    appearance_embedding_size: int = 1
    geo_feat_dim: int = 15
    num_layers: int = 2
    num_layers_color: int = 3
    num_proposal_samples_per_ray: Tuple[int, ...] = (256, 96)
    num_nerf_samples_per_ray: int = 48
    num_proposal_iterations: int = 2
    proposal_update_every: int = 5
    proposal_warmup: int = 5000
    use_same_proposal_network: bool = False
    proposal_net_args_list: List[dict] = [
        {"hidden_dim": 16, "log2_hashmap_size": 17, "num_levels": 5, "max_res": 128},
        {"hidden_dim": 16, "log2_hashmap_size": 17, "num_levels": 5, "max_res": 256},
    ]
    proposal_weights_anneal_slope: float = 10.0
    proposal_weights_anneal_max_num_iters: int = 1000
    use_proposal_weight_anneal: bool = True
    use_single_jitter: bool = True
    interlevel_loss_mult: float = 1.0
    distortion_loss_mult: float = 0.002
    disable_scene_contraction: bool = False
    background_color: Literal["black", "white", "last_sample"] = "last_sample"
    train_near_far: List[float] = [0.05, 1e3]
    aabb_norm_range: Union[List[float], torch.Tensor] = [0, 1]
    white_bkgd: bool = False
    camera: str = "normal"
    patch_size: int = 128
    add_upsample: int = -1
    add_lpips: int = -1
    runtime: Literal["Torch", "Kernel"] = "Kernel"
    lr_init: float = 1e-2
    lr: Optional[float] = None                      # the reference's spelling (nerfacto.py:95); wins when given
    lr_final: float = 0.0001
    lr_decay_max_steps: int = 50000
    eps: float = 1e-15
    # the "path" split of the datasets (fly-around or trajectory file)
    render_px: int = 720
    render_fov: float = 65.0
    render_nframes: int = 100
    render_skip: int = 1
    render_fps: int = 30
    render_spherical: bool = False
    render_spherical_zdiff: float = 1.0
    render_spherical_radius: float = 4.0
    render_downward: float = -45.0
    render_ncircle: float = 1
    render_path: bool = False
    render_pathid: int = 0
    render_near_far: Optional[List[float]] = None
    render_lb: Optional[List[float]] = None
    render_ub: Optional[List[float]] = None
    render_batch_size: int = 8192
    distance_scale: float = 25
    render_stratified_sampling: bool = False        # the reference jitters evaluation renders too (True there)

    @model_validator(mode="after")
    def _one_spelling(self):
        """Both spellings of the two renamed fields read the same value afterwards."""
        if self.appearance_embed_dim is not None:
            self.appearance_embedding_dim = int(self.appearance_embed_dim)
        self.appearance_embed_dim = self.appearance_embedding_dim
        if self.lr is not None:
            self.lr_init = float(self.lr)
        self.lr = self.lr_init
        return self


def scene_contraction(x: torch.Tensor) -> torch.Tensor:
    """L-infinity contraction onto the cube of half-width 2: identity inside the unit cube,
    ``(2 - 1/|x|) x / |x|`` outside (with the infinity norm)."""
    mag = x.abs().amax(dim=-1, keepdim=True).clamp_min(1e-9)
    return torch.where(mag <= 1, x, (2 - 1 / mag) * (x / mag))


class Nerfacto(BaseNeRF):
    def __init__(self, aabb, device, near_far, scene_manager=None, config=None, group=None):
        super().__init__(config=config, scene_manager=scene_manager, aabb=aabb, device=device, near_far=list(near_far))
        self.aabb = torch.as_tensor(aabb, dtype=torch.float32, device=device)
        self.group = group
        self.plane_division = config.get("plane_division", [1, 1]) or [1, 1]
        self.num_hash_table = int(self.plane_division[0] * self.plane_division[1])
        self.step = 0
        self.init_field_components()
        self.init_sampler()
        self.init_renderer()

    def init_field_components(self):
        c = self.config
        self.geo_feat_dim = c.geo_feat_dim
        self.contract = None if c.disable_scene_contraction else scene_contraction
        self.direction_encoding = SHEncoding(levels=4)
        n_tables = 1 if (c.get("branch_parallel", False) and c.get("is_train", False)) else self.num_hash_table
        self.mlp_base_grid = HashEncoding(c.num_levels, c.base_res, c.max_res, c.log2_hashmap_size,
                                          c.features_per_level, device=self.device, num_hash_table=n_tables)
        self.mlp_base_mlp = MLPDecoder(self.mlp_base_grid.get_out_dim(), c.hidden_dim, c.num_layers,
                                       1 + self.geo_feat_dim, None, mlp_bias=False).to(self.device)
        self.mlp_head = MLPDecoder(self.direction_encoding.get_out_dim() + self.geo_feat_dim + c.appearance_embedding_dim,
                                   c.hidden_dim_color, c.num_layers_color, 3, nn.Sigmoid(), mlp_bias=False).to(self.device)
        self.embedding_appearance = nn.Embedding(c.appearance_embedding_size, c.appearance_embedding_dim).to(self.device)
        if c.get("runtime", "Torch") == "Kernel":
            self.mlp_base_mlp.use_fused = self.mlp_head.use_fused = True

    def init_sampler(self):
        c = self.config
        self.proposal_networks = ProposalNetworks(self.aabb.cpu(), c.num_proposal_iterations, c.proposal_net_args_list,
                                                  c.use_same_proposal_network, self.contract, device=self.device).to(self.device)

        def update_schedule(step):
            return int(np.clip(np.interp(step, [0, c.proposal_warmup], [0, c.proposal_update_every]), 1,
                               c.proposal_update_every))

        self.sampler = ProposalNetworkSampler(c.num_proposal_samples_per_ray, c.num_nerf_samples_per_ray,
                                              c.num_proposal_iterations, c.use_single_jitter, update_schedule,
                                              c.proposal_weights_anneal_max_num_iters, c.proposal_weights_anneal_slope,
                                              c.use_proposal_weight_anneal)

    def init_renderer(self):
        self.renderer = VolumeRenderer(white_bg=self.config.white_bkgd)

    def _positions(self, pos: torch.Tensor):
        if self.contract is not None:
            unit = (pos - self.aabb[0]) / (self.aabb[1] - self.aabb[0]) * 2.0 - 1.0
            norm = (self.contract(unit) + 2.0) / 4.0
        else:
            norm = (pos - self.aabb[0]) / (self.aabb[1] - self.aabb[0])
        inside = ((norm > 0.0) & (norm < 1.0)).all(dim=-1)
        if self.num_hash_table == 1:
            return torch.cat((norm * inside[:, None], torch.zeros_like(norm[:, :1])), -1), inside
        nx, ny = self.plane_division
        u, v = norm[:, 0] * nx, norm[:, 1] * ny
        bx, by = u.floor().clamp(0, nx - 1), v.floor().clamp(0, ny - 1)
        block, inside = window_block_ids(self.scene_manager, bx, by, nx, ny, inside)
        local = torch.stack((u - bx, v - by, norm[:, 2]), -1) * inside[:, None]
        c = self.config
        if c.get("branch_parallel", False) and c.get("is_train", False):
            mine = block == float(c.mp_rank)
            inside, block, local = inside & mine, torch.zeros_like(block), local * mine[:, None]
        return torch.cat((local, block[:, None]), -1), inside

    def _mp_sum(self, t):
        c = self.config
        if c.get("branch_parallel", False) and c.get("is_train", False):
            from ...comm.autograd import all_reduce_sum_local_grad

            return all_reduce_sum_local_grad(t, c.mp_group)
        return t

    def _kernel_glue(self, rays) -> bool:
        """Kernel path for the per-sample glue: both field heads on the fused MLP kernels and no cross-rank sum between
        the density head and the colour head (spatial-block training sums the two across ranks there)."""
        c = self.config
        if not rays.is_cuda or (c.get("branch_parallel", False) and c.get("is_train", False)):
            return False
        if not (getattr(self.mlp_base_mlp, "use_fused", False) and getattr(self.mlp_head, "use_fused", False)):
            return False
        from ...ops import native
        from ...ops.fused_mlp import fused_mlp_supported

        return (native.available() and self.geo_feat_dim + c.appearance_embedding_dim <= 48
                and fused_mlp_supported(self.mlp_base_mlp) and fused_mlp_supported(self.mlp_head))

    def get_density(self, pos: torch.Tensor, directions: Optional[torch.Tensor] = None,
                    z_vals: Optional[torch.Tensor] = None):
        """``(density [N, 1], geometry features [N, G])`` at world positions ``pos [N, 3]``; with the reference's
        arguments ``(origins, directions, z_vals)`` the positions are ``origins + directions * z_vals[..., None]``."""
        if directions is not None and z_vals is not None:
            lead = pos.shape[:-1]
            pos = (pos + directions * z_vals[..., None]).reshape(-1, 3)
            sigma, geo = self.get_density(pos)
            return sigma.reshape(*lead, 1), geo.reshape(*lead, -1)
        xyzb, inside = self._positions(pos)
        h = self.mlp_base_mlp(self.mlp_base_grid(xyzb)).float()
        raw, geo = torch.split(h, [1, self.geo_feat_dim], dim=-1)
        return self._mp_sum(trunc_exp(raw) * inside[:, None]), self._mp_sum(geo * inside[:, None])

    @property
    def proposal_sampler(self):
        """The proposal sampler under the reference's attribute name (nerfacto.py:168)."""
        return self.sampler

    def step_cb(self, step: int) -> None:
        """Per-iteration callback of the sampler's update schedule and annealing."""
        self.sampler.step_cb(step)

    def density_fn(self, positions: torch.Tensor) -> torch.Tensor:
        """Density only, at world positions ``[..., 3]`` (reference: nerfacto.py:228-236)."""
        return self.get_density(positions.reshape(-1, 3))[0].reshape(*positions.shape[:-1], 1)

    def set_anneal(self, step: int) -> float:
        """Proposal-weight annealing of mip-NeRF 360 (eq. 18) at ``step``, handed to the sampler (reference:
        nerfacto.py:339-353)."""
        c = self.config
        self.step = step
        frac = float(np.clip(step / max(c.proposal_weights_anneal_max_num_iters, 1), 0, 1))
        b = c.proposal_weights_anneal_slope
        anneal = b * frac / ((b - 1) * frac + 1)
        self.sampler.set_anneal(anneal)
        return anneal

    def forward(self, rays_chunk):
        c = self.config
        rays = rays_chunk.data if isinstance(rays_chunk, Rays) else rays_chunk
        o, d = rays[:, :3].contiguous(), rays[:, 3:6].contiguous()
        cam = rays[:, 6] if rays.shape[1] > 6 else torch.zeros(rays.shape[0], device=rays.device)
        self.sampler.train(self.training)
        near, far = self.near_far
        samples, weights_list, samples_list = self.sampler(
            o, d, near, far, self.proposal_networks.density_fns, cam,
            render_stratified_sampling=bool(c.get("render_stratified_sampling", False)))
        R, S = samples.starts.shape[:2]
        pos = samples.positions.reshape(-1, 3)
        if self.training:
            app_ray = self.embedding_appearance(cam.long().clamp(0, c.appearance_embedding_size - 1))
        else:
            app_ray = self.embedding_appearance.weight.mean(0)[None, :].expand(R, -1)           # mean embedding at eval
        if self._kernel_glue(rays):
            # sigma (truncated exp) and the colour head's bf16 rows [SH(dir) | geometry | appearance] in one launch from the
            # density head's output, one launch for the backward of both (ops/csrc/ngp_field.cu)
            from ...ops import ngp_field

            xyzb, inside = self._positions(pos)
            h = self.mlp_base_mlp(self.mlp_base_grid(xyzb)).float()
            width = (16 + self.geo_feat_dim + c.appearance_embedding_dim + 15) // 16 * 16
            rows, sigma = ngp_field.head_rows(None, S, d, h, inside, app_ray.contiguous(), c.appearance_embedding_dim, width)
            density = sigma[:, None]
            rgb = self.mlp_head(rows).float().view(R, S, 3)
        else:
            density, geo = self.get_density(pos)
            dirs = get_normalized_directions(d)[:, None, :].expand(-1, S, -1).reshape(-1, 3)
            app = app_ray[:, None, :].expand(-1, S, -1).reshape(-1, c.appearance_embedding_dim)
            rgb = self.mlp_head(torch.cat((self.direction_encoding(dirs), geo, app), dim=-1)).float().view(R, S, 3)
        weights = samples.get_weights(density.view(R, S, 1))
        weights_list.append(weights)
        samples_list.append(samples)
        z = 0.5 * (samples.starts + samples.ends)[..., 0]
        bg = 1.0 if (c.white_bkgd or c.background_color == "white") else 0.0
        rgb_map, depth_map, acc = composite_render(weights[..., 0].contiguous(), rgb, z.contiguous(), bg)
        if c.background_color == "last_sample" and not c.white_bkgd:
            rgb_map = rgb_map + (1.0 - weights[..., 0].sum(-1, keepdim=True)) * rgb[:, -1, :]
        out = {"rgb_map": rgb_map.clamp(0, 1), "depth_map": depth_map.unsqueeze(-1)}
        if self.training:
            out["weights_list"], out["ray_samples_list"] = weights_list, samples_list
        return out

    def get_optparam_groups(self, lr: Optional[float] = None):
        lr = self.config.lr_init if lr is None else lr
        return [{"params": list(self.mlp_base_grid.parameters()) + list(self.mlp_base_mlp.parameters())
                 + list(self.mlp_head.parameters()) + list(self.embedding_appearance.parameters()), "lr": lr, "name": "fields"},
                {"params": list(self.proposal_networks.parameters()), "lr": lr, "name": "proposal_networks"}]

    def kwargs(self):
        return {"aabb": self.aabb, "device": self.device, "near_far": self.near_far}

    def merge_ckpts(self, ckpt_fp_list, kwargs_fp_list, map_location="cpu"):
        from ..instant_ngp.instant_ngp import InstantNGP

        return InstantNGP.merge_ckpts(self, ckpt_fp_list, kwargs_fp_list, map_location)

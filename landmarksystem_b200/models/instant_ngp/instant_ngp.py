"""InstantNGP: multiresolution hash grid + tiny MLPs + occupancy-grid marching (reference:
benchmarks/nerf/instant_ngp/instant_ngp.py:24-454)."""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Union

import torch
from torch import nn
from typing_extensions import Literal

from ...components.data.rays import Rays
from ...components.fields.encodings.hash_encoding import HashEncoding
from ...components.fields.encodings.sh_encoding import SHEncoding
from ...components.fields.mlp_decoder import MLPDecoder
from ...components.model.base_model import BaseNeRF
from ...components.ray_samplers.volumetric_sampler import VolumetricSampler
from ...components.renderers import VolumeRenderer
from ...components.utils.activation_utils import trunc_exp
from ...configs import ConfigClass
from ...ops.occgrid import OccGridEstimator


class InstantNGPConfig(ConfigClass):
    num_levels: int = 16
    base_res: int = 16
    max_res: int = 2048
    log2_hashmap_size: int = 19
    features_per_level: int = 2
    hidden_dim: int = 64
    hidden_dim_color: int = 64
    appearance_embedding_dim: int = 32
    appearance_embedding_size: int = 1
    geo_feat_dim: int = 15
    num_layers: int = 2
    num_layers_color: int = 3
    grid_resolution: int = 128
    grid_levels: int = 4
    alpha_thre: float = 0.01
    cone_angle: float = 0.004
    render_step_size: Optional[float] = None
    max_samples_per_ray: int = 256
    background_color: Literal["black", "white"] = "white"
    train_near_far: List[float] = [0.05, 1e3]
    aabb_norm_range: Union[List[float], torch.Tensor] = [0, 1]
    white_bkgd: bool = False
    camera: str = "normal"
    patch_size: int = 128
    add_upsample: int = -1
    add_lpips: int = -1
    runtime: Literal["Torch", "Kernel"] = "Kernel"
    lr_init: float = 1e-2
    lr_final: float = 0.0001
    lr_decay_max_steps: int = 200000
    eps: float = 1e-15
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
    render_stratified_sampling: bool = True


def get_normalized_positions(pos: torch.Tensor, aabb: torch.Tensor) -> torch.Tensor:
    return (pos - aabb[0]) / (aabb[1] - aabb[0])


def get_normalized_directions(dirs: torch.Tensor) -> torch.Tensor:
    return (dirs / dirs.norm(dim=-1, keepdim=True) + 1.0) / 2.0


class _FieldDensity:
    """The density callback handed to the occupancy sampler: positions -> sigma, and - for the sampler's opacity culling on
    the kernel path - marched intervals -> sigma without materialising gathered positions (sample index -> hash-grid
    coordinate by ``ngp_positions_kernel``, then the density head)."""

    def __init__(self, model):
        self.model = model

    def __call__(self, positions):
        return self.model.density_fn(positions)

    @torch.no_grad()
    def from_samples(self, idx, samples_per_ray, origins, directions, t_starts, t_ends):
        m = self.model
        z = (0.5 * (t_starts + t_ends)).reshape(-1).contiguous().float()
        if not m._kernel_glue(origins):
            flat = idx if idx is not None else torch.arange(z.numel(), device=z.device)
            ray = flat // samples_per_ray
            return m.density_fn(origins[ray] + directions[ray] * z[flat][:, None]).reshape(-1)
        from ...ops import ngp_field

        xyzb, inside = ngp_field.sample_positions(idx, samples_per_ray, origins.contiguous().float(),
                                                  directions.contiguous().float(), z, m.aabb, m._aabb_host,
                                                  int(m.plane_division[0]), int(m.plane_division[1]))
        single = m.mlp_base_grid.num_hash_table == 1
        if not single:
            xyzb, inside = window_remap(m.scene_manager, xyzb, inside, int(m.plane_division[0]), int(m.plane_division[1]))
        feat = m.mlp_base_grid(xyzb, out_dtype=torch.bfloat16) if single else m.mlp_base_grid(xyzb)
        h = m.mlp_base_mlp(feat)
        # the step's own forward evaluates the survivors of the culling at the same positions with the same weights:
        # it takes the features and the head's output from here instead of looking them up again
        m._cull_cache = {"feat": feat, "h": h} if (single and m.training) else None
        return torch.exp(h[:, 0].float()) * inside


def window_block_ids(scene_manager, bx: torch.Tensor, by: torch.Tensor, nx: int, ny: int, inside: torch.Tensor):
    """Table index of every sample from its block coordinates ``(bx, by)``.  With the whole scene resident that is the
    row-major block id; under dynamic loading only a window of ``local_block_partition`` blocks is resident, its tables
    sit in window order, and samples outside the window are masked (the reference indexes tables by the window-relative
    ``block_idx`` of ``SceneManager.assign_blockIdx``, benchmarks/nerf/instant_ngp/instant_ngp.py:239-255)."""
    local = getattr(scene_manager, "local_block_partition", None)
    if scene_manager is None or local is None or [int(local[0]), int(local[1])] == [int(nx), int(ny)]:
        return bx * ny + by, inside
    lx, ly = int(local[0]), int(local[1])
    rx, ry = bx - scene_manager.relative_block_idx_x, by - scene_manager.relative_block_idx_y
    within = (rx >= 0) & (rx < lx) & (ry >= 0) & (ry < ly)
    return torch.where(within, rx * ly + ry, torch.zeros_like(rx)), inside & within


def window_remap(scene_manager, xyzb: torch.Tensor, inside: torch.Tensor, nx: int, ny: int):
    """:func:`window_block_ids` applied to ``[M, 4]`` rows that carry the row-major block id in their last column (the
    output of the position kernel); rows outside the resident window are zeroed and masked."""
    local = getattr(scene_manager, "local_block_partition", None)
    if scene_manager is None or local is None or [int(local[0]), int(local[1])] == [int(nx), int(ny)]:
        return xyzb, inside
    block = xyzb[:, 3]
    bx, by = torch.div(block, ny, rounding_mode="floor"), torch.remainder(block, ny)
    rel, keep = window_block_ids(scene_manager, bx, by, nx, ny, inside)
    return torch.cat((xyzb[:, :3] * keep[:, None], rel[:, None]), -1), keep


class InstantNGP(BaseNeRF):
    def __init__(self, aabb, device, near_far, scene_manager=None, config=None, group=None):
        super().__init__(config=config, scene_manager=scene_manager, aabb=aabb, device=device, near_far=list(near_far))
        self.aabb = torch.as_tensor(aabb, dtype=torch.float32, device=device)
        self.group = group
        self.plane_division = config.get("plane_division", [1, 1]) or [1, 1]
        self.num_hash_table = int(self.plane_division[0] * self.plane_division[1])
        if config.render_step_size is None:
            config.render_step_size = float(((self.aabb[1] - self.aabb[0]) ** 2).sum().sqrt()) / 1000
        self.step = 0
        self._aabb_host = [float(v) for v in self.aabb.reshape(-1).tolist()]
        self.init_field_components()
        self.init_sampler()
        self.init_renderer()

    # -- construction ------------------------------------------------------------------------------------
    def init_field_components(self):
        c = self.config
        self.geo_feat_dim = c.geo_feat_dim
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
        self.occupancy_grid = OccGridEstimator(torch.cat((self.aabb[0], self.aabb[1])).cpu(), c.grid_resolution,
                                               c.grid_levels).to(self.device)
        self.sampler = VolumetricSampler(self.occupancy_grid, _FieldDensity(self), self.near_far, c.render_step_size,
                                         c.alpha_thre, c.cone_angle, c.max_samples_per_ray)

    def init_renderer(self):
        self.renderer = VolumeRenderer(white_bg=self.config.white_bkgd)

    # -- field --------------------------------------------------------------------------------------------------
    def _positions(self, pos: torch.Tensor):
        """World positions -> ``([N, 4] hash-grid input: block-local xyz in [0, 1] + block id, inside mask)``."""
        norm = get_normalized_positions(pos, self.aabb)
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
            inside = inside & mine
            block = torch.zeros_like(block)
            local = local * mine[:, None]
        return torch.cat((local, block[:, None]), -1), inside

    def _cached_field_rows(self, idx, samples_per_ray: int):
        """Rows of the sampler's density query (this step, same weights) that belong to the samples ``idx`` that
        survived the culling: ``(hash features bf16 [M, L*F], density-head output fp32 [M, 1+G])`` or ``(None, None)``."""
        cache, self._cull_cache = getattr(self, "_cull_cache", None), None
        cull = getattr(self.occupancy_grid, "last_cull", None)
        if cache is None or cull is None or not torch.is_grad_enabled():
            return None, None
        feat, h = cache["feat"], cache["h"]
        if feat.shape[0] != cull["n_queried"]:
            return None, None
        if idx.numel() == cull["n_queried"]:
            return feat, h                          # nothing was culled; the compaction keeps the order
        from ...ops import ngp_field

        where = None
        if cull["queried"] is not None:           # the query covered a subset of the slots: flat slot -> row of the query
            where = torch.full((cull["source"].numel(),), -1, dtype=torch.long, device=idx.device)
            where[cull["queried"]] = torch.arange(cull["n_queried"], device=idx.device)
        return ngp_field.gather_cached_rows(idx, samples_per_ray, cull["source"], where, feat, h)

    def _kernel_glue(self, rays) -> bool:
        """The per-sample glue runs as kernels when both heads are on the fused MLP path and no cross-rank sum sits
        between the density head and the colour head (spatial-block training sums the two across ranks there)."""
        c = self.config
        if not rays.is_cuda or (c.get("branch_parallel", False) and c.get("is_train", False)):
            return False
        if not (getattr(self.mlp_base_mlp, "use_fused", False) and getattr(self.mlp_head, "use_fused", False)):
            return False
        from ...ops import native

        return native.available() and self.geo_feat_dim + c.appearance_embedding_dim <= 48

    def _mp_sum(self, t):
        c = self.config
        if c.get("branch_parallel", False) and c.get("is_train", False):
            from ...comm.autograd import all_reduce_sum_local_grad

            return all_reduce_sum_local_grad(t, c.mp_group)
        return t

    def get_density(self, origins, directions, z_vals):
        pos = origins + directions * z_vals
        xyzb, inside = self._positions(pos)
        h = self.mlp_base_mlp(self.mlp_base_grid(xyzb)).float()
        raw, geo = torch.split(h, [1, self.geo_feat_dim], dim=-1)
        density = trunc_exp(raw) * inside[:, None]
        # branch parallel: each sample was evaluated by the one rank that owns its block
        return self._mp_sum(density), self._mp_sum(geo * inside[:, None])

    def density_fn(self, positions):
        return self.get_density(positions, torch.zeros_like(positions), torch.zeros_like(positions[..., :1]))[0]

    def update_occupancy_grid(self, step: int):
        import torch.distributed as dist

        c = self.config
        self.occupancy_grid.update_every_n_steps(step=step, occ_eval_fn=lambda x: self.density_fn(x) * c.render_step_size)
        if (c.get("branch_parallel", False) or c.get("DDP", False)) and dist.is_initialized() and step % 16 == 0 \
                and self.occupancy_grid.training:
            dist.broadcast(self.occupancy_grid.occs, src=0)
            occs = self.occupancy_grid.occs
            self.occupancy_grid.binaries = (occs > torch.clamp(occs.mean(), max=0.01)).view(self.occupancy_grid.binaries.shape)

    # -- forward ----------------------------------------------------------------------------------------------------
    def forward(self, rays_chunk):
        c = self.config
        rays = rays_chunk.data if isinstance(rays_chunk, Rays) else rays_chunk
        self.sampler.train(self.training)
        o, dvec, ts, te, valid = self.sampler(rays, training=self.training,
                                              render_stratified_sampling=c.render_stratified_sampling, lean=True)
        R, S = valid.shape
        idx = valid.reshape(-1).nonzero(as_tuple=True)[0]
        z_vals = 0.5 * (ts + te)
        sigma = torch.zeros(R * S, device=rays.device)
        rgb = torch.zeros(R * S, 3, device=rays.device)
        if idx.numel() > 0 and self._kernel_glue(rays):
            # kernel path: positions -> hash-grid coordinates in one launch; sigma and the colour head's bf16 input rows
            # (SH | geometry | appearance) in one launch from the density head's output; one backward launch for both
            from ...ops import ngp_field

            full = idx.numel() == R * S
            kidx = None if full else idx
            o32, d32 = o.contiguous().float(), dvec.contiguous().float()
            xyzb, inside = ngp_field.sample_positions(kidx, S, o32, d32, z_vals.reshape(-1).contiguous().float(), self.aabb,
                                                      self._aabb_host, int(self.plane_division[0]), int(self.plane_division[1]))
            feat_pre, h_pre = self._cached_field_rows(idx, S)
            if self.mlp_base_grid.num_hash_table > 1:
                xyzb, inside = window_remap(self.scene_manager, xyzb, inside, int(self.plane_division[0]),
                                            int(self.plane_division[1]))
            if self.mlp_base_grid.num_hash_table == 1:
                # bf16 rows straight from the lookup kernel: what the head kernel reads and its backward returns
                feat = self.mlp_base_grid(xyzb, out_dtype=torch.bfloat16, precomputed=feat_pre)
            else:
                feat = self.mlp_base_grid(xyzb)
            h = self.mlp_base_mlp(feat, precomputed=h_pre).float()
            per_ray = None
            if self.training:
                cam = rays[:, 6] if rays.shape[1] > 6 else torch.zeros(R, device=rays.device)
                per_ray = self.embedding_appearance(cam.long().clamp(0, c.appearance_embedding_size - 1))
            width = (16 + self.geo_feat_dim + c.appearance_embedding_dim + 15) // 16 * 16
            rows, sig = ngp_field.head_rows(kidx, S, d32, h, inside, per_ray, c.appearance_embedding_dim, width)
            color = self.mlp_head(rows).float()
            if full:
                sigma, rgb = sig, color
            else:
                sigma = sigma.index_put((idx,), sig)
                rgb = rgb.index_put((idx,), color)
        elif idx.numel() > 0:
            # positions and directions of the valid samples only (no packed [R, S, 13] sample block)
            ray = idx // S
            dirs = dvec[ray]
            xyz = o[ray] + dirs * z_vals.reshape(-1)[idx][:, None]
            density, geo = self.get_density(xyz, torch.zeros_like(xyz), torch.zeros_like(xyz[:, :1]))
            d = self.direction_encoding(get_normalized_directions(dirs))
            if self.training:
                # one embedding row per RAY, gathered per sample: the embedding's backward then reduces R rows instead
                # of sorting R x S sample indices
                cam = rays[:, 6] if rays.shape[1] > 6 else torch.zeros(R, device=rays.device)
                per_ray = self.embedding_appearance(cam.long().clamp(0, c.appearance_embedding_size - 1))
                app = per_ray[ray]
            else:
                app = torch.zeros(idx.numel(), c.appearance_embedding_dim, device=rays.device)
            color = self.mlp_head((d, geo, app)).float()
            sigma = sigma.index_put((idx,), density[:, 0])
            rgb = rgb.index_put((idx,), color)
        dists = (te - ts) * valid
        weight = self.renderer.get_weights(sigma.view(R, S), dists)
        white = 1.0 if (c.white_bkgd or c.background_color == "white") else 0.0
        from ...ops import composite_render

        rgb_map, depth_map, _ = composite_render(weight, rgb.view(R, S, 3), z_vals, white)
        return {"rgb_map": rgb_map.clamp(0, 1), "depth_map": depth_map.unsqueeze(-1)}

    # -- optimisation / checkpoints -----------------------------------------------------------------------------------
    def get_optparam_groups(self):
        lr = self.config.lr_init
        return [{"params": list(self.mlp_base_grid.parameters()), "lr": lr},
                {"params": list(self.mlp_base_mlp.parameters()), "lr": lr},
                {"params": list(self.mlp_head.parameters()), "lr": lr},
                {"params": list(self.embedding_appearance.parameters()), "lr": lr}]

    def kwargs(self):
        return {"aabb": self.aabb, "device": self.device, "near_far": self.near_far}

    def merge_ckpts(self, ckpt_fp_list, kwargs_fp_list, map_location="cpu"):
        states = [torch.load(fp, map_location=map_location, weights_only=False) for fp in ckpt_fp_list]
        kwargs = torch.load(kwargs_fp_list[0], map_location=map_location, weights_only=False)
        merged = OrderedDict()
        for key in states[0].keys():
            if key.startswith("mlp_base_grid.") and key.endswith("params"):
                for i, sd in enumerate(states):
                    merged[key.replace("tcnn_encoding.params", f"tcnn_encoding.{i}.params")] = sd[key]
            else:
                merged[key] = states[0][key]
        return merged, kwargs

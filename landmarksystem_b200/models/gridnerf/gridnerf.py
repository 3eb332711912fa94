"""GridNeRF: VM feature grids + tiny MLP heads, rendered by volume compositing.

Model-zoo counterpart of the reference's ``benchmarks/nerf/gridnerf/gridnerf.py`` (config :33-134,
decoder heads :137-197, model :200-928).  Same configuration fields, parameter names and checkpoint
keys; the forward pass is organised around flat ``[R*S]`` sample tensors that feed the channels-last
lookup kernel, the fused MLP and the warp-scan compositor instead of masked gathers over a packed
sample struct.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn
from typing_extensions import Literal

from ...components.data.rays import Rays
from ...components.fields.alpha_mask import AlphaGridMask
from ...components.fields.embedding import AppearanceEmbedding
from ...components.fields.encodings.base_encoding import VolumeEncoding
from ...components.fields.encodings.tensor_vm_encoding import TensorVMEncoding
from ...components.fields.mlp_decoder import MLPDecoder, positional_encoding
from ...components.fields.nerf_branch import NeRF, raw2outputs
from ...components.model.base_model import BaseNeRF
from ...components.ray_samplers import PDFSampler, UniformSampler
from ...components.renderers import VolumeRenderer
from ...components.utils.loss_utils import eff_distloss
from ...configs import ConfigClass


class GridNeRFConfig(ConfigClass):
    """Model hyper-parameters (field names follow the reference config, gridnerf.py:33-134)."""

    resMode: List[int] = [1]
    encode_app: bool = False
    run_nerf: bool = False
    nerf_D: int = 6
    nerf_D_a: int = 2
    nerf_W: int = 128
    nerf_freq: int = 16
    n_importance: int = 128
    nerf_n_importance: int = 16
    nonlinear_density: bool = False
    fea2denseAct: str = "relu"
    n_lamb_sigma: List[int] = [16, 16, 16]
    n_lamb_sh: List[int] = [48, 48, 48]
    data_dim_color: int = 27
    pos_pe: int = 6
    view_pe: int = 6
    fea_pe: int = 6
    featureC: int = 128
    density_shift: float = -10
    ndims: int = 1
    appearance_embedding_size: int = 1
    add_upsample: int = -1
    add_lpips: int = -1
    add_nerf: int = -1
    add_distort: int = -1
    patch_size: int = 128
    residnerf: bool = False
    train_near_far: list = [0.1, 10.0]
    lr_init: float = 0.02
    lr_basis: float = 1e-3
    lr_decay_iters: int = -1
    lr_decay_target_ratio: float = 0.1
    lr_upsample_reset: bool = True
    L1_weight_inital: float = 0.0
    L1_weight_rest: float = 0.0
    Ortho_weight: float = 0.0
    TV_weight_density: float = 0.0
    TV_weight_app: float = 0.0
    alpha_mask_thre: float = 0.0001
    nSamples: int = int(1e6)
    step_ratio: float = 0.5
    N_voxel_init: int = 100 ** 3
    N_voxel_final: int = 300 ** 3
    upsamp_list: list = []
    update_AlphaMask_list: list = []
    progressive_alpha: int = 0
    alpha_grid_reso: int = 256 ** 3
    rayMarch_weight_thres: float = 0.001
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
    render_near_far: Optional[list] = None
    render_lb: Optional[list] = None
    render_ub: Optional[list] = None
    render_batch_size: int = 8192
    distance_scale: float = 25
    sampling_opt: bool = False
    alpha_mask_filter_thre: float = 0
    white_bkgd: bool = False
    dynamic_fetching: bool = False
    neighbour_size: int = 9
    camera: str = "normal"
    rm_weight_mask_thre: float = 0.0
    runtime: Literal["Torch", "Kernel"] = "Torch"
    # additions of this framework (defaults keep the reference behaviour)
    grid_dtype: Literal["fp32", "bf16"] = "fp32"  # bf16: kernels read bf16 shadows of fp32 master grids
    init_grid_size: Optional[list] = None         # explicit [nx, ny, nz] voxel grid instead of N_voxel_init
    fused_mlp_train: bool = False                 # colour head through the tcgen05 kernel while training too
    branch_dispatch: Literal["allreduce", "a2a"] = "allreduce"   # a2a: every rank brings its own rays; samples
                                                  # travel to the GPU owning their block over NVLink peer memory
    fused_optimizer: bool = True
    deterministic_grid_grad: bool = False         # atomic-free sorted backward of the grid lookup (bit-reproducible, slower)
    fused_sampler: bool = True                    # sampling + block assignment in one kernel on CUDA
    fused_density: bool = True                    # density lookup + head in one kernel on CUDA
    lazy_adam: bool = False                       # deferred (exact) Adam on the planes: visit touched texels only

    def check_args(self) -> None:
        super().check_args()
        assert self.ndims in (1, 2, 3)
        assert self.fea2denseAct in ("relu", "softplus")


class RGBDecoder(nn.Module):
    """``basis_mat`` projection of the appearance feature, sin/cos encodings of it and of the view
    direction, then a 3-layer MLP with a sigmoid (reference: gridnerf.py:137-174)."""

    def __init__(self, n_component, resMode, app_dim, view_pe=6, fea_pe=6, featureC=128, encode_app=False) -> None:
        super().__init__()
        self.basis_mat = nn.Linear(sum(n_component) * len(resMode), app_dim, bias=False)
        self.encode_app, self.viewpe, self.feape, self.app_dim = encode_app, view_pe, fea_pe, app_dim
        in_mlp = 2 * max(view_pe, 0) * 3 + 2 * fea_pe * app_dim + 3 * (view_pe > -1) + app_dim + (48 if encode_app else 0)
        self.decoder = MLPDecoder(inChanel=in_mlp, layer_width=featureC, num_layers=3, out_dim=3,
                                  out_activation=nn.Sigmoid())

    def forward(self, samples_dir, app_features, app_latent=None):
        if app_features.is_cuda and app_latent is None and getattr(self, "use_fused", False):
            from ...ops.fused_mlp import rgb_decoder_forward, rgb_decoder_supported

            if rgb_decoder_supported(self):
                return rgb_decoder_forward(self, samples_dir, app_features)
        f = self.basis_mat(app_features.to(self.basis_mat.weight.dtype))
        parts = [f]
        if self.encode_app and app_latent is not None:
            parts.append(app_latent)
        if self.viewpe > -1:
            parts.append(samples_dir)
        if self.feape > 0:
            parts.append(positional_encoding(f, self.feape))
        if self.viewpe > 0:
            parts.append(positional_encoding(samples_dir, self.viewpe))
        return self.decoder(torch.cat(parts, dim=-1))


class _ShiftedSoftplus(nn.Module):
    def __init__(self, shift: float):
        super().__init__()
        self.shift = shift

    def forward(self, x):
        return F.softplus(x + self.shift)


class Feature2Density(nn.Module):
    """Density head (reference: gridnerf.py:177-197).  The reference's softplus branch appends a
    lambda to ``nn.Sequential``, which cannot run; a proper shifted-softplus module is used here."""

    def __init__(self, sum_n_component, resModeLen, nonlinear_density, density_shift, fea2denseAct):
        super().__init__()
        layers = []
        if nonlinear_density:
            layers += [nn.Linear(sum_n_component * resModeLen, 1, bias=False), nn.ReLU()]
        self.nonlinear = nonlinear_density
        layers.append(nn.ReLU() if fea2denseAct == "relu" else _ShiftedSoftplus(density_shift))
        self.feature2density = nn.Sequential(*layers)

    def forward(self, sigma_feature):
        if not self.nonlinear:
            sigma_feature = sigma_feature.sum(dim=-1, keepdim=True)
        return self.feature2density(sigma_feature)

    def kernel_args(self):
        """``(weight or None, inner_relu, activation name, shift)`` for the fused lookup + head kernel."""
        last = self.feature2density[-1]
        weight = self.feature2density[0].weight if self.nonlinear else None
        if isinstance(last, _ShiftedSoftplus):
            return weight, self.nonlinear, "softplus", float(last.shift)
        return weight, self.nonlinear, "relu", 0.0


def n_to_reso(n_voxels, bbox):
    xyz_min, xyz_max = bbox
    voxel = ((xyz_max - xyz_min).prod() / n_voxels).pow(1 / len(xyz_min))
    return ((xyz_max - xyz_min) / voxel).long().tolist()


def cal_n_samples(reso, step_ratio=0.5):
    return int(np.linalg.norm(reso) / step_ratio)


class GridNeRF(BaseNeRF):
    def __init__(self, aabb, gridSize, device, alphaMask=None, near_far=(2.0, 6.0), scene_manager=None,
                 grid_shape=None, config=None):
        super().__init__(config, scene_manager, aabb=aabb, gridSize=gridSize, device=device, alphaMask=alphaMask,
                         grid_shape=grid_shape, near_far=list(near_far))
        self.aabb = torch.as_tensor(aabb, dtype=torch.float32, device=device)
        self.run_nerf = config.run_nerf
        if bool(config.get("deterministic_grid_grad", False)):
            from ...ops import vm

            vm.DETERMINISTIC_BACKWARD = True        # process-wide: atomic-free sorted backward of every grid lookup
        self.density_n_comp = config.n_lamb_sigma[: config.ndims]
        self.app_n_comp = config.n_lamb_sh[: config.ndims]
        self.app_dim = config.data_dim_color
        self.plane_division = getattr(config, "plane_division", [1, 1])
        self.sigma_batch = self.app_batch = self.nerf_batch = None
        self.update_stepSize(gridSize)
        self.init_field_components()
        self.init_sampler()
        self.init_renderer()

    # -- construction -------------------------------------------------------------------
    def init_sampler(self):
        self.sampler = UniformSampler(num_samples=self.nSamples, step_size=self.stepSize, aabb=self.aabb,
                                      near_far=self.near_far)
        self.pdf_sampler = PDFSampler(num_samples=self.config.nerf_n_importance)

    def _local_blocks(self) -> int:
        sm = self.scene_manager
        if getattr(self.config, "branch_parallel", False) and getattr(self.config, "is_train", False):
            return 1  # each model-parallel rank owns exactly one spatial block
        return sm.n_local_blocks if sm is not None else 1

    def init_field_components(self):
        cfg = self.config
        part = self.scene_manager.block_partition.tolist() if self.scene_manager is not None else [1, 1]
        grid = [int(v) for v in self.gridSize]
        grid[0], grid[1] = grid[0] // part[0], grid[1] // part[1]
        n_blocks = self._local_blocks()
        shapes = self.grid_shape or {}
        fill = not bool(cfg.get("grids_come_from_ckpt", False))
        self.density_encoding = TensorVMEncoding(cfg.ndims, cfg.resMode, cfg.n_lamb_sigma, grid, self.device,
                                                 param_shape=shapes.get("density_encoding"), n_blocks=n_blocks, random_init=fill)
        self.rgb_encoding = TensorVMEncoding(cfg.ndims, cfg.resMode, cfg.n_lamb_sh, grid, self.device,
                                             param_shape=shapes.get("rgb_encoding"), n_blocks=n_blocks, random_init=fill)
        self.feature2density = Feature2Density(sum(self.density_encoding.n_component), len(cfg.resMode),
                                               cfg.nonlinear_density, cfg.density_shift, cfg.fea2denseAct).to(self.device)
        self.rgb_decoder = RGBDecoder(self.rgb_encoding.n_component, cfg.resMode, self.app_dim, cfg.view_pe,
                                      cfg.fea_pe, cfg.featureC, cfg.encode_app).to(self.device)
        if cfg.encode_app:
            self.embedding_app = AppearanceEmbedding(cfg.appearance_embedding_size, self.app_n_comp[0], self.device)
        if cfg.add_nerf > 0 or self.run_nerf:
            self.init_nerf()
        if cfg.grid_dtype == "bf16" and torch.device(self.device).type == "cuda":
            self.enable_shadow()

    def enable_shadow(self):
        cfg = self.config
        # the deferred update is exact only when every gradient comes from sample lookups, i.e. no dense
        # regulariser (L1 / TV over whole planes) is active
        dense_reg = any(float(cfg.get(k, 0.0) or 0.0) > 0 for k in
                        ("L1_weight_inital", "L1_weight_rest", "TV_weight_density", "TV_weight_app", "Ortho_weight"))
        lazy = bool(cfg.get("lazy_adam", False)) and not dense_reg
        self.density_encoding.enable_shadow(self.config.fused_optimizer, lazy)
        self.rgb_encoding.enable_shadow(self.config.fused_optimizer, lazy)

    def use_shadow(self) -> bool:
        return bool(self.density_encoding.use_shadow)

    def refresh_shadow(self):
        self.density_encoding.refresh_shadow()
        self.rgb_encoding.refresh_shadow()

    def init_renderer(self):
        self.renderer = VolumeRenderer(white_bg=self.config.white_bkgd)

    def init_nerf(self):
        cfg = self.config
        self.nerf = NeRF(cfg, sum(self.density_n_comp) * len(cfg.resMode),
                         sum(self.app_n_comp) * len(cfg.resMode)).to(self.device)
        self.residnerf = cfg.residnerf
        self.nerf_n_importance = cfg.nerf_n_importance

    def channel_last(self):
        self.density_encoding.channel_last()
        self.rgb_encoding.channel_last()

    def update_stepSize(self, gridSize):
        cfg = self.config
        self.aabbSize = self.aabb[1] - self.aabb[0]
        self.invaabbSize = 2.0 / self.aabbSize
        self.gridSize = torch.as_tensor([int(v) for v in gridSize], device=self.aabb.device)
        self.units = self.aabbSize / (self.gridSize - 1)
        self.stepSize = float(torch.mean(self.units) * cfg.step_ratio)
        self.aabbDiag = float(torch.sqrt(torch.sum(torch.square(self.aabbSize))))
        self.nSamples = int(self.aabbDiag / self.stepSize) + 1

    # -- field queries ------------------------------------------------------------------
    def _xyzb(self, xyz: torch.Tensor, valid: Optional[torch.Tensor] = None) -> torch.Tensor:
        """World xyz ``[N, 3]`` -> kernel coordinates ``[N, 4]`` (block-local xyz, block id or -1)."""
        local, block = self.scene_manager.block_local_coords(self.scene_manager.normalize_coord(xyz))
        if valid is not None:
            block = torch.where(valid, block, torch.full_like(block, -1.0))
        if getattr(self.config, "branch_parallel", False) and getattr(self.config, "is_train", False):
            # this rank stores only its own block (index 0 locally); others are looked up remotely
            mine = block == float(self.config.mp_rank)
            self._owner = block
            block = torch.where(mine, torch.zeros_like(block), torch.full_like(block, -1.0))
        return torch.cat((local, block[:, None]), dim=-1)

    # -- branch parallel through the peer-memory all-to-all -------------------------------------------------
    def _use_a2a(self) -> bool:
        c = self.config
        return bool(c.get("branch_parallel", False) and c.get("is_train", False) and c.get("branch_dispatch") == "a2a"
                    and self.aabb.is_cuda and torch.distributed.is_initialized())

    def _dispatcher(self, n_rows: int):
        disp = getattr(self, "_a2a", None)
        if disp is None or disp.cap < n_rows:
            from ...parallel.branch_dispatch import BlockDispatcher

            if disp is not None:
                disp.close()                 # every rank outgrows the capacity at the same call

            disp = BlockDispatcher(n_rows, max_w=6, max_v=3, group=self.config.mp_group)
            self._a2a = disp
        return disp

    class _OwnerFn:
        """Callable evaluated on the owning rank; exposes the parameters its backward feeds."""

        def __init__(self, model, kind):
            self.model, self.kind = model, kind

        def parameters_for_autograd(self):
            m = self.model
            mods = [m.density_encoding, m.feature2density] if self.kind == "sigma" else [m.rgb_encoding, m.rgb_decoder]
            return [p for mod in mods for p in mod.parameters()]

        accepts_route = True       # the dispatcher may hand over the rows' return route

        def __call__(self, coords, extra, m_dev, route=None):
            """``coords [M_cap, 4]`` / ``extra [M_cap, 3]`` hold ``m_dev`` (device int) received rows; the result has
            ``M_cap`` rows of which the first ``m_dev`` are valid.  Kernel paths never learn ``m_dev`` on the host.
            ``route``: where each row's result has to go; when the kernel path stores the results there itself,
            ``self.combined`` is set and the dispatcher skips its own combine kernel."""
            m = self.model
            self.combined = False
            if self.kind == "sigma":
                m.sigma_batch = m_dev
                enc = m.density_encoding
                if bool(m.config.get("fused_density", True)) and enc.fused_density_ok(coords):
                    self.combined = route is not None
                    return m._density(coords, count=m_dev, route=route)[:, None]
                k = int(m_dev.item())
                return F.pad(m._density(coords[:k])[:, None], (0, 0, 0, coords.shape[0] - k))
            m.app_batch = m_dev
            if m._fused_app_stage_ok(coords):
                from ...ops.fused_mlp import RGB_IN_WIDTH, rgb_decoder_forward

                # the lookup kernel writes the directions behind the features: rows leave it complete
                feat = m.rgb_encoding(coords, count=m_dev, out_dtype=torch.bfloat16, out_width=RGB_IN_WIDTH, zero_fill=False,
                                      tail=(extra.contiguous().float(), None, 1, 144))
                return rgb_decoder_forward(m.rgb_decoder, None, feat, m_dev)
            k = int(m_dev.item())
            return F.pad(m._rgb(coords[:k], extra[:k].contiguous(), None), (0, 0, 0, coords.shape[0] - k))

    def _density(self, xyzb: torch.Tensor, count=None, route=None) -> torch.Tensor:
        enc, head = self.density_encoding, self.feature2density
        if bool(self.config.get("fused_density", True)) and hasattr(enc, "fused_density_ok") and enc.fused_density_ok(xyzb):
            return enc.density(xyzb, *head.kernel_args(), count=count, route=route)
        feat = enc(xyzb, count=count) if count is not None else enc(xyzb)
        return head(feat).squeeze(-1).float()

    def _rgb(self, xyzb, dirs, app_latent=None) -> torch.Tensor:
        dec = self.rgb_decoder
        fused_ok = (not torch.is_grad_enabled()) or bool(self.config.get("fused_mlp_train", False))
        if (fused_ok and xyzb.is_cuda and app_latent is None and getattr(dec, "use_fused", False)
                and self.config.ndims == 1
                and type(self.rgb_encoding).__name__ in ("TensorVMEncoding", "BranchParallelTensorVMEncoding",
                                                         "FusedTensorVMEncoding")):
            from ...ops.fused_mlp import RGB_IN_WIDTH, rgb_decoder_supported

            if rgb_decoder_supported(dec):
                # lookup writes bf16 rows straight into the fused decoder's 160-wide input layout
                feat = self.rgb_encoding(xyzb, out_dtype=torch.bfloat16, out_width=RGB_IN_WIDTH)
                return dec(dirs, feat, None).float()
        feat = self.rgb_encoding(xyzb)
        return dec(dirs, feat, app_latent).float()

    # -- colour stage on compacted rows, no host synchronisation ------------------------------------------
    def _fused_app_stage_ok(self, xyzb: torch.Tensor) -> bool:
        dec = self.rgb_decoder
        if not (xyzb.is_cuda and getattr(dec, "use_fused", False) and not self.config.encode_app and self.config.ndims == 1
                and type(self.rgb_encoding).__name__ in ("TensorVMEncoding", "BranchParallelTensorVMEncoding",
                                                         "FusedTensorVMEncoding")):
            return False
        from ...ops.fused_mlp import rgb_backward_supported, rgb_decoder_supported

        if not rgb_decoder_supported(dec):
            return False
        if not torch.is_grad_enabled():
            return True
        return bool(self.config.get("fused_mlp_train", False)) and rgb_backward_supported(dec)

    def _fused_app_stage(self, xyzb, dirs, app_mask, samples_per_ray: int) -> torch.Tensor:
        """Samples above the weight threshold are compacted on the device (count stays there), looked up,
        decoded by the tcgen05 colour head and scattered back to ``[R*S, 3]``: the reference's
        ``nonzero`` + gathers + ``index_put`` (benchmarks/nerf/gridnerf/gridnerf.py:846-871) without the
        host round trip, with static shapes."""
        from ...ops.fused_mlp import RGB_IN_WIDTH, rgb_decoder_forward
        from ...ops.select import ScatterRows3, compact_rows

        idx, coords, count = compact_rows(app_mask, xyzb)
        self.app_batch = count
        # the colour head reads only the feature and direction columns of the first `count` rows
        feat = self.rgb_encoding(coords, count=count, out_dtype=torch.bfloat16, out_width=RGB_IN_WIDTH, zero_fill=False,
                                 tail=(dirs.contiguous().float(), idx, samples_per_ray, 144))
        vals = rgb_decoder_forward(self.rgb_decoder, None, feat, count)
        return ScatterRows3.apply(vals, idx, coords, count, xyzb.shape[0])

    def compute_alpha(self, xyz_locs: torch.Tensor, length: float = 1.0) -> torch.Tensor:
        valid = None
        if self.alphaMask is not None:
            valid = self.alphaMask.sample_alpha(xyz_locs) > 0
        sigma = self._density(self._xyzb(xyz_locs, valid))
        sigma = self._mp_sum(sigma)
        return 1.0 - torch.exp(-sigma * length)

    def _mp_sum(self, t: torch.Tensor) -> torch.Tensor:
        """Branch parallel: every sample is evaluated by exactly one rank (zeros elsewhere), so the
        exchange of the reference's ``sync_sigma``/``sync_rgb`` is a sum over the MP group whose
        backward is the identity on the local contribution."""
        if getattr(self.config, "branch_parallel", False) and getattr(self.config, "is_train", False):
            from ...comm.autograd import all_reduce_sum_local_grad

            return all_reduce_sum_local_grad(t, self.config.mp_group)
        return t

    @torch.no_grad()
    def getDenseAlpha(self, gridSize=None, with_xyz: bool = True):
        """Alpha of one step at every vertex of a ``gridSize`` lattice over the scene box, evaluated slab by slab;
        ``with_xyz=False`` returns only ``alpha [X, Y, Z]`` and never builds the dense coordinate tensor."""
        gridSize = [int(v) for v in (self.gridSize if gridSize is None else gridSize)]
        lin = [torch.linspace(0, 1, g, device=self.aabb.device) for g in gridSize]
        if with_xyz:
            samples = torch.stack(torch.meshgrid(*lin, indexing="ij"), -1)
            dense_xyz = self.aabb[0] * (1 - samples) + self.aabb[1] * samples
        else:
            yz = torch.stack(torch.meshgrid(lin[1], lin[2], indexing="ij"), -1).reshape(-1, 2)
        alpha = torch.zeros(gridSize, device=self.aabb.device)
        for i in range(gridSize[0]):
            if with_xyz:
                pts = dense_xyz[i].reshape(-1, 3)
            else:
                s = torch.cat((lin[0][i].expand(yz.shape[0], 1), yz), -1)
                pts = self.aabb[0] * (1 - s) + self.aabb[1] * s
            alpha[i] = self.compute_alpha(pts, self.stepSize).view(gridSize[1], gridSize[2])
        return (alpha, dense_xyz) if with_xyz else alpha

    @torch.no_grad()
    def updateAlphaMask(self, gridSize=(200, 200, 200), increase_alpha_thresh=0):
        cfg = self.config
        gridSize = [int(v) for v in gridSize]
        from ...ops.resize import alpha_mask_pool

        alpha = self.getDenseAlpha(gridSize, with_xyz=False)
        thre = cfg.alpha_mask_thre * (10 ** increase_alpha_thresh)
        # clamp, 3x3x3 max-pool, threshold, transpose to [Z, Y, X] and the occupied index box in one pass
        mask, bbox = alpha_mask_pool(alpha, thre)
        self.alphaMask = AlphaGridMask(self.device, self.aabb, mask)
        bbox = bbox.tolist()
        if bbox[3] < 0:
            return self.aabb.clone()
        denom = torch.tensor([max(g - 1, 1) for g in gridSize], device=self.aabb.device, dtype=self.aabb.dtype)
        lo = torch.tensor(bbox[:3], device=self.aabb.device, dtype=self.aabb.dtype) / denom
        hi = torch.tensor(bbox[3:], device=self.aabb.device, dtype=self.aabb.dtype) / denom
        return torch.stack((self.aabb[0] * (1 - lo) + self.aabb[1] * lo, self.aabb[0] * (1 - hi) + self.aabb[1] * hi))

    def distortion_loss(self, weight, z_vals, dists):
        mids = 0.5 * (z_vals[:, 1:] + z_vals[:, :-1])
        m = torch.cat((mids, mids[:, -1:]), dim=-1)
        return 0.01 * eff_distloss(weight, m, dists).unsqueeze(0)

    # -- forward --------------------------------------------------------------------------
    def _grid_pass(self, rays: torch.Tensor, n_samples: int, hull: bool, app_code=None):
        """One sampling + density + weights + colour + composite pass over ``rays [R, 7]``."""
        cfg = self.config
        train = bool(cfg.is_train)
        S_req = n_samples if n_samples > 0 else self.sampler.num_samples
        a2a = self._use_a2a()
        mp_train = bool(getattr(cfg, "branch_parallel", False)) and train
        fused_front = (rays.is_cuda and not (hull and train) and self.alphaMask is None and self.scene_manager is not None
                       and bool(cfg.get("fused_sampler", True)) and (a2a or not mp_train) and not cfg.encode_app)
        origin, dirs = rays[:, :3], rays[:, 3:6]
        if fused_front:
            # sampling, box test, block assignment and block-local coordinates in one kernel
            from ...ops.sampler import uniform_sample_blocks

            sm = self.scene_manager
            jitter = torch.rand(rays.shape[0], device=rays.device) if train else None
            z, dists, xyzb, valid = uniform_sample_blocks(
                rays, S_req, self.aabb, float(self.sampler.near_far[0]), float(self.sampler.near_far[1]),
                float(self.sampler.step_size), sm._norm_lo, sm.aabb_norm_size, sm._partition,
                (sm.relative_block_idx_x, sm.relative_block_idx_y), tuple(sm.local_block_partition), jitter, hull=hull)
            R, S = z.shape
            if a2a:
                disp = self._dispatcher(R * S)
                sigma = disp.query(xyzb, None, GridNeRF._OwnerFn(self, "sigma"), 1, channel=f"sigma{int(hull)}",
                                   payload_width=3, owner_column=3).view(R, S)
            else:
                self.sigma_batch = None
                sigma = self._mp_sum(self._density(xyzb)).view(R, S)
        else:
            z = self.sampler.compute_z_vals(rays, S_req, train, hull)
            R, S = z.shape
            xyz = (origin[:, None, :] + dirs[:, None, :] * z[..., None]).reshape(-1, 3)
            valid = ~((xyz < self.aabb[0]) | (xyz > self.aabb[1])).any(dim=-1)
            if self.alphaMask is not None:
                valid = valid & (self.alphaMask.sample_alpha(xyz) > cfg.alpha_mask_filter_thre)
            if a2a:
                local, block = self.scene_manager.block_local_coords(self.scene_manager.normalize_coord(xyz))
                owner = torch.where(valid, block, torch.full_like(block, -1.0))
                xyzb = torch.cat((local, owner[:, None]), dim=-1)
                disp = self._dispatcher(R * S)
                sigma = disp.query(local, owner, GridNeRF._OwnerFn(self, "sigma"), 1, channel=f"sigma{int(hull)}").view(R, S)
            else:
                xyzb = self._xyzb(xyz, valid)
                self.sigma_batch = (xyzb[:, 3] >= 0).sum()
                sigma = self._mp_sum(self._density(xyzb)).view(R, S)
            dists = torch.cat((z[:, 1:] - z[:, :-1], torch.zeros_like(z[:, :1])), dim=-1)
        weight = self.renderer.get_weights(sigma, dists * cfg.distance_scale)
        app_mask = (weight > cfg.rayMarch_weight_thres).reshape(-1)
        rgb = torch.zeros(R * S, 3, device=rays.device, dtype=torch.float32)
        if a2a:
            from ...ops.select import ScatterRows3, build_payload6, compact_rows

            idx, coords_c, count = compact_rows(app_mask, xyzb)          # stays on the device: no row count reaches the host
            payload, owner_c = build_payload6(coords_c, dirs, idx, count, S)
            vals = self._dispatcher(R * S).query(payload, owner_c, GridNeRF._OwnerFn(self, "rgb"), 3, count=count,
                                                 channel=f"rgb{int(hull)}")
            rgb = ScatterRows3.apply(vals, idx, coords_c, count, R * S)
            rgb_map, depth_map = self.renderer(weight, rgb.view(R, S, 3), z, 0.5 if self.training else 0.0)
            return rgb_map, depth_map, weight, app_mask.view(R, S), z, dists
        if self._fused_app_stage_ok(xyzb):
            rgb = self._fused_app_stage(xyzb, dirs, app_mask, S)
            rgb = self._mp_sum(rgb)
            rgb_map, depth_map = self.renderer(weight, rgb.view(R, S, 3), z, 0.5 if self.training else 0.0)
            return rgb_map, depth_map, weight, app_mask.view(R, S), z, dists
        idx = app_mask.nonzero(as_tuple=True)[0]
        self.app_batch = (xyzb[idx, 3] >= 0).sum()
        if idx.numel() > 0 or (train and getattr(cfg, "branch_parallel", False)):
            if idx.numel() == 0:
                idx = torch.zeros(1, dtype=torch.long, device=rays.device)  # keep every rank's graph alive
            ray_of = idx // S
            latent = None
            if cfg.encode_app:
                cam = rays[ray_of, 6].long() if app_code is None else None
                latent = self.embedding_app(cam, xyz[idx], app_code)
            vals = self._rgb(xyzb[idx], dirs[ray_of], latent)
            vals = vals * (xyzb[idx, 3:4] >= 0).to(vals.dtype)
            rgb = rgb.index_put((idx,), vals)
        rgb = self._mp_sum(rgb)
        rgb_map, depth_map = self.renderer(weight, rgb.view(R, S, 3), z, 0.5 if self.training else 0.0)
        return rgb_map, depth_map, weight, app_mask.view(R, S), z, dists

    def forward(self, rays_chunk, app_code=None, N_samples=-1):
        cfg = self.config
        rays = rays_chunk.data if isinstance(rays_chunk, Rays) else rays_chunk
        outputs = {}
        dense = cfg.is_train or not cfg.sampling_opt
        if dense:
            rgb_map, depth_map, weight, app_mask, z, dists = self._grid_pass(rays, N_samples, False, app_code)
            if not cfg.is_train:
                outputs = (rgb_map, depth_map)
            else:
                outputs = {"rgb_map": rgb_map, "depth_map": depth_map,
                           "distort_loss": self.distortion_loss(weight * app_mask, z, dists)}
        if (not cfg.is_train and cfg.sampling_opt) or (cfg.is_train and self.run_nerf):
            rgb_map, depth_map, weight, app_mask, z, dists = self._grid_pass(rays, cfg.n_importance, True, app_code)
            if not cfg.is_train:
                return rgb_map, depth_map
            outputs.update({"rgb_map1": rgb_map, "depth_map1": depth_map,
                            "distort_loss1": self.distortion_loss(weight * app_mask, z, dists)})
            outputs.update(self._nerf_pass(rays, z, weight, rgb_map, app_code))
        return outputs

    def _nerf_pass(self, rays, z, weight, rgb_map, app_code):
        cfg = self.config
        samples = self.pdf_sampler(rays, z, weight[..., 1:-1].detach(), self.nerf_n_importance)
        R, S = samples.shape
        xyz = samples.xyz.reshape(-1, 3)
        xyzb = self._xyzb(xyz)
        self.nerf_batch = (xyzb[:, 3] >= 0).sum()
        latent = self.embedding_app(samples.camera_idx.reshape(-1), xyz, app_code) if cfg.encode_app else None
        den_feat = self.density_encoding(xyzb)
        app_feat = self.rgb_encoding(xyzb)
        raw = self.nerf(xyz, samples.dirs.reshape(-1, 3), den_feat, app_feat, latent).float()
        raw = self._mp_sum(raw * (xyzb[:, 3:4] >= 0).to(raw.dtype)).view(R, S, 4)
        extras = raw2outputs(raw, samples.dists)
        depth = (extras["weights"] * samples.z_vals).sum(-1)
        rgb = (extras["rgb_map"] + rgb_map).clamp(0.0, 1.0) if self.residnerf else extras["rgb_map"]
        return {"rgb_map_nerf": rgb, "depth_map_nerf": depth}

    @torch.no_grad()
    def render_partial(self, rays: torch.Tensor, N_samples: int = -1) -> torch.Tensor:
        """Model-parallel rendering, per-rank half: composite only the samples that fall into THIS rank's resident
        blocks (the scene manager's window) and return ``[R, 8]`` records ``(rgb without background, transmittance,
        depth, opacity, entry distance, 0)``.  Records of all ranks are merged in entry-distance order by
        :class:`landmarksystem_b200.parallel.composite_merge.CompositeMerger`; the result equals the single-model
        render as long as a ray crosses each rank's region in one contiguous interval (rectangular block windows)."""
        from ...ops.composite import composite_render, composite_weights
        from ...parallel.composite_merge import pack_partial

        cfg = self.config
        hull = bool(cfg.sampling_opt)                     # same sampling as the single-model render of this configuration
        S_req = cfg.n_importance if hull else (N_samples if N_samples > 0 else self.sampler.num_samples)
        origin, dirs = rays[:, :3], rays[:, 3:6]
        sm = self.scene_manager
        if rays.is_cuda and self.alphaMask is None and bool(cfg.get("fused_sampler", True)):
            from ...ops.sampler import uniform_sample_blocks

            z, dists, xyzb, _ = uniform_sample_blocks(
                rays, S_req, self.aabb, float(self.sampler.near_far[0]), float(self.sampler.near_far[1]),
                float(self.sampler.step_size), sm._norm_lo, sm.aabb_norm_size, sm._partition,
                (sm.relative_block_idx_x, sm.relative_block_idx_y), tuple(sm.local_block_partition), None, hull=hull)
            R, S = z.shape
            mine = xyzb[:, 3] >= 0
        else:
            z = self.sampler.compute_z_vals(rays, S_req, False, hull)
            R, S = z.shape
            xyz = (origin[:, None, :] + dirs[:, None, :] * z[..., None]).reshape(-1, 3)
            valid = ~((xyz < self.aabb[0]) | (xyz > self.aabb[1])).any(dim=-1)
            if self.alphaMask is not None:
                valid = valid & (self.alphaMask.sample_alpha(xyz) > cfg.alpha_mask_filter_thre)
            local, block = sm.block_local_coords(sm.normalize_coord(xyz))
            block = torch.where(valid, block, torch.full_like(block, -1.0))
            xyzb = torch.cat((local, block[:, None]), dim=-1)
            mine = (block >= 0)
            dists = torch.cat((z[:, 1:] - z[:, :-1], torch.zeros_like(z[:, :1])), dim=-1)
        sigma = (self._density(xyzb) * mine.to(torch.float32)).view(R, S)      # softplus heads are not zero at no-data
        weight, trans = composite_weights(sigma, dists * cfg.distance_scale)
        app_mask = ((weight > cfg.rayMarch_weight_thres) & mine.view(R, S)).reshape(-1)
        if self._fused_app_stage_ok(xyzb):
            rgb = self._fused_app_stage(xyzb, dirs, app_mask, S)
        else:
            rgb = torch.zeros(R * S, 3, device=rays.device, dtype=torch.float32)
            idx = app_mask.nonzero(as_tuple=True)[0]
            if idx.numel() > 0:
                rgb = rgb.index_put((idx,), self._rgb(xyzb[idx], dirs[idx // S], None))
        rgb_map, depth, acc = composite_render(weight, rgb.view(R, S, 3), z, 0.0)
        t_entry = torch.where(mine.view(R, S), z, torch.full_like(z, float("inf"))).amin(dim=-1)
        return pack_partial(rgb_map, trans, depth, acc, t_entry)

    def render_all_rays(self, rays, chunk_size: Optional[int] = None, N_samples=-1, idxs=None, app_code=0):
        n_total = rays.shape[0]
        chunk_size = chunk_size or n_total
        if idxs is None:
            idxs = torch.zeros(n_total, device=rays.device)
        collected = {}
        for start in range(0, n_total, chunk_size):
            chunk = rays[start:start + chunk_size]
            if chunk.shape[-1] == 6:
                chunk = torch.cat((chunk, idxs[start:start + chunk_size, None].to(chunk.dtype)), dim=-1)
            ret = self.forward(chunk, N_samples=N_samples)
            if not isinstance(ret, dict):
                ret = {"rgb_map": ret[0], "depth_map": ret[1]}
            for key, value in ret.items():
                collected.setdefault(key, []).append(value)
        return {k: torch.cat(v, 0) for k, v in collected.items()}

    # -- optimisation ----------------------------------------------------------------------
    def get_optparam_groups(self, lr_init_spatial=0.02, lr_init_network=0.001):
        groups = [
            {"params": list(self.density_encoding.parameters()), "lr": lr_init_spatial},
            {"params": list(self.rgb_encoding.parameters()), "lr": lr_init_spatial},
            {"params": list(self.feature2density.parameters()), "lr": lr_init_network},
            {"params": list(self.rgb_decoder.parameters()), "lr": lr_init_network},
        ]
        if self.config.encode_app:
            groups.append({"params": list(self.embedding_app.parameters()), "lr": lr_init_network})
        if self.run_nerf or hasattr(self, "nerf"):
            groups.append({"params": list(self.nerf.parameters()), "lr": 5e-4})
        return [g for g in groups if len(g["params"]) > 0]

    @torch.no_grad()
    def upsample_volume_grid(self, res_target):
        part = self.scene_manager.block_partition.tolist()
        grid = [int(v) for v in res_target]
        grid[0], grid[1] = grid[0] // part[0], grid[1] // part[1]
        self.density_encoding.upsample_volume_grid(grid)
        self.rgb_encoding.upsample_volume_grid(grid)
        self.update_stepSize(res_target)
        self.sampler.step_size = self.stepSize
        self.sampler.num_samples = self.nSamples

    # -- checkpoints ---------------------------------------------------------------------------
    def kwargs(self):
        kw = super().kwargs()
        kw["aabb"] = self.aabb
        kw["gridSize"] = self.gridSize.tolist()
        kw["alphaMask"] = self.alphaMask
        return kw

    def merge_ckpts(self, ckpt_fp_list, kwargs_fp_list, map_location="cpu"):
        """Merge per-rank ``state_dict-sub{r}.th`` files into one block-stacked state dict and the
        matching kwargs (with ``grid_shape``), as written by branch-parallel training."""
        states = [torch.load(fp, map_location=map_location, weights_only=False) for fp in ckpt_fp_list]
        kwargs = torch.load(kwargs_fp_list[0], map_location=map_location, weights_only=False)
        merged, grid_shape = OrderedDict(), OrderedDict()
        for name, module in self.named_children():
            keys = [k for k in states[0].keys() if k.split(".")[0] == name]
            if isinstance(module, VolumeEncoding):
                part = module.merge_state_dicts([{k: sd[k] for k in keys} for sd in states], device=map_location)
                merged.update(part)
                grid_shape[name] = {k[len(name) + 1:]: list(v.shape) for k, v in part.items()}
            else:
                for k in keys:
                    merged[k] = states[0][k]
        kwargs["grid_shape"] = grid_shape
        return merged, kwargs

    def edit_model(self, edit_mode: dict):
        return None

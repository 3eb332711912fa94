"""GridNeRF trainer: schedule, losses, checkpointing and evaluation.

Counterpart of the reference's ``benchmarks/nerf/gridnerf/gridnerf_trainer.py`` (create_model
:65-125, optimiser :127-164, train loop :166-527, evaluation :529-718).  Launch:
``torchrun --nproc-per-node N -m landmarksystem_b200.models.gridnerf.gridnerf_trainer --config conf.py [--key value]``.
"""
from __future__ import annotations

import os
import sys
import time
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ...components.data.data_manager import DatasetManager
from ...components.scene import SceneManager
from ...components.utils.image_utils import mse2psnr_npy, visualize_depth_numpy
from ...components.utils.loss_utils import rgb_ssim
from ...configs import BaseConfig, get_default_parser, parse_console_args
from ...convertor import ComponentConvertorFactory
from ...ops import FusedAdam
from ...parallel.grad_sync import GradSynchronizer
from ...train.nerf_trainer import NeRFTrainer
from ...train.utils import is_main_rank
from .gridnerf import GridNeRF, cal_n_samples, n_to_reso


def save_image(path: str, array: np.ndarray) -> None:
    from PIL import Image

    Image.fromarray(array).save(path)


class GridNeRFTrainer(NeRFTrainer):
    def __init__(self, config):
        super().__init__(config)
        self.init_train_env()
        self.check_args()
        self.scene_mgr = SceneManager(self.config)
        self.data_mgr = DatasetManager(self.config)
        self.iteration = config.start_iters
        self.create_model()
        self.create_optimizer()
        self._init_schedule()

    def check_args(self):
        super().check_args()
        cfg = self.config
        if cfg.branch_parallel:
            assert cfg.plane_division[0] * cfg.plane_division[1] == cfg.model_parallel_degree

    # -- model / optimiser ---------------------------------------------------------------------
    def create_model(self):
        cfg = self.config
        aabb = self.scene_mgr.aabb.to(cfg.device)
        self.scene_mgr.to(cfg.device)
        ckpt, kwargs_fp = self._resume_paths()
        if kwargs_fp is not None and os.path.exists(kwargs_fp):
            kwargs = GridNeRF.get_kwargs_from_ckpt(kwargs_fp, cfg.device)
            kwargs.update(device=cfg.device, scene_manager=self.scene_mgr, config=cfg)
            model = GridNeRF(**kwargs)
            model.load_from_state_dict(model.get_state_dict_from_ckpt(ckpt, cfg.device), strict=False)
            if model.use_shadow():
                model.refresh_shadow()
        else:
            reso = list(cfg.init_grid_size) if cfg.get("init_grid_size") else n_to_reso(cfg.N_voxel_init, aabb)
            near_far = list(self.data_mgr.dataset_info.near_far)
            model = GridNeRF(aabb, reso, cfg.device, near_far=near_far, scene_manager=self.scene_mgr, config=cfg)
        self.module = model
        if cfg.model_parallel:
            model = ComponentConvertorFactory.get_convertor("parallelize").convert(model, cfg)
        if cfg.get("runtime", "Torch") == "Kernel":
            model = ComponentConvertorFactory.get_convertor("runtime").convert(model, cfg)
        self.model = self.module = model
        # replicated parameters are synchronised explicitly between backward and the optimiser step
        on_gpu = torch.device(cfg.device).type == "cuda"
        self.mp_sync = GradSynchronizer(cfg.mp_group, average=False, p2p_small=on_gpu) if cfg.branch_parallel else None
        self.dp_sync = GradSynchronizer(cfg.dp_group if cfg.model_parallel else None, average=True) if cfg.DDP else None
        return model

    def _resume_paths(self):
        cfg = self.config
        ckpt = cfg.get("ckpt")
        if ckpt == "auto":
            suffix = f"-sub{cfg.rank}" if cfg.model_parallel else ""
            ckpt = f"{self.logfolder}/state_dict{suffix}.th"
            if not os.path.exists(ckpt):
                return None, None
        if not ckpt:
            return None, None
        kwargs_fp = cfg.get("kwargs") or ckpt.replace("state_dict", "kwargs")
        return ckpt, kwargs_fp

    def _replicated_params(self):
        m = self.module
        mods = [m.feature2density, m.rgb_decoder]
        if self.config.encode_app:
            mods.append(m.embedding_app)
        if hasattr(m, "nerf"):
            mods.append(m.nerf)
        return [p for mod in mods for p in mod.parameters()]

    def _make_optimizer(self, groups):
        """Adam over ``groups``.  CUDA + data parallel: gradient reduce-scatter, partitioned Adam and parameter
        all-gather fused in one peer-memory kernel per learning-rate group; CUDA single replica: fused
        Adam; CPU: ``torch.optim.Adam``."""
        cfg = self.config
        on_cuda = torch.device(cfg.device).type == "cuda"
        decay = cfg.lr_decay_target_ratio ** (1.0 / (cfg.lr_decay_iters if cfg.lr_decay_iters > 0 else cfg.n_iters))
        for g in groups:
            g["lr_decay"] = decay              # per-step factor; fused optimisers need it to reconstruct / advance the schedule
        if on_cuda and cfg.DDP and cfg.get("dp_optimizer", "p2p_zero") == "p2p_zero" and dist.is_initialized():
            from ...parallel.zero_adam import GroupedP2PZeroAdam

            self.dp_sync = None        # the fused kernel does the reduction
            return GroupedP2PZeroAdam(groups, betas=(0.9, 0.99), group=cfg.dp_group if cfg.model_parallel else None,
                                      shadow=cfg.get("grid_dtype") == "bf16")
        use_fused = bool(cfg.get("fused_optimizer", True)) and on_cuda
        if use_fused:
            return FusedAdam(groups, betas=(0.9, 0.99), capturable=bool(cfg.get("cuda_graph", False)))
        return torch.optim.Adam(groups, betas=(0.9, 0.99))

    def create_optimizer(self):
        cfg = self.config
        groups = self.module.get_optparam_groups(cfg.lr_init, cfg.lr_basis)
        self.optimizer = self._make_optimizer(groups)
        optim_file = self._optim_path()
        if cfg.get("ckpt") and os.path.exists(optim_file):
            self.optimizer.load_state_dict(torch.load(optim_file, map_location=cfg.device, weights_only=False)["optimizer"])
        return self.optimizer

    def _optim_path(self):
        """Model-parallel ranks and ranks of a partitioned (ZeRO) optimiser each own different state and write their own
        file; replicas of an ordinary optimiser share rank 0's."""
        cfg = self.config
        per_rank = cfg.model_parallel or bool(getattr(self.optimizer, "partitioned", False))
        suffix = f"-sub{cfg.rank}" if per_rank else ""
        return os.path.join(self.optim_dir, f"{cfg.expname}_opt{suffix}.th")

    def save_optimizer(self, path: Optional[str] = None):
        """``{"optimizer": state_dict}`` at ``path`` (default: this run's ``optim/{expname}_opt[-sub{r}].th``)."""
        os.makedirs(self.optim_dir, exist_ok=True)
        torch.save({"optimizer": self.optimizer.state_dict()}, path or self._optim_path())

    def _replace_optimizer(self, groups):
        """New optimiser over ``groups`` (parameters were replaced or added); the old one's peer-mapped buffers are
        released first - a collective teardown, reached by every rank at the same iteration."""
        old = getattr(self, "optimizer", None)
        if old is not None and hasattr(old, "close"):
            old.close()
        self.optimizer = self._make_optimizer(groups)
        return self.optimizer

    def _group_lr(self, params, default):
        """Current learning rate of the optimiser group holding ``params`` (fused optimisers merge groups by rate)."""
        opt = self.optimizer
        if hasattr(opt, "group_lr"):
            return opt.group_lr(params)
        for g in opt.param_groups:
            if any(p is params[0] for p in g["params"]):
                return g["lr"]
        return default

    # -- schedule ---------------------------------------------------------------------------
    def _init_schedule(self):
        cfg = self.config
        decay_iters = cfg.lr_decay_iters if cfg.lr_decay_iters > 0 else cfg.n_iters
        self.lr_factor = cfg.lr_decay_target_ratio ** (1.0 / decay_iters)
        n_up = len(cfg.upsamp_list)
        self.n_voxel_list = torch.round(torch.exp(torch.linspace(
            np.log(cfg.N_voxel_init), np.log(cfg.N_voxel_final), n_up + 1))).long().tolist()[1:]
        self.tv_weight_density, self.tv_weight_app = cfg.TV_weight_density, cfg.TV_weight_app
        self.l1_weight = cfg.L1_weight_inital
        self.enable_distort = False
        self.nsamples = min(int(cfg.nSamples), cal_n_samples(self.module.gridSize.tolist(), cfg.step_ratio))
        # replay the upsampling schedule when resuming
        for it, n_vox in zip(cfg.upsamp_list, self.n_voxel_list):
            if cfg.start_iters > it and not cfg.get("ckpt"):
                self._upsample(n_vox)

    def _upsample(self, n_voxels):
        cfg = self.config
        reso = n_to_reso(n_voxels, self.module.aabb)
        self.nsamples = min(int(cfg.nSamples), cal_n_samples(reso, cfg.step_ratio))
        self.module.upsample_volume_grid(reso)
        lr_scale = 1.0 if cfg.lr_upsample_reset else cfg.lr_decay_target_ratio ** (self.iteration / cfg.n_iters)
        groups = self.module.get_optparam_groups(cfg.lr_init * lr_scale, cfg.lr_basis * lr_scale)
        self._replace_optimizer(groups)                # parameters were replaced: new state

    # -- one optimisation step -------------------------------------------------------------------
    def compute_loss(self, all_ret, rgb_train):
        cfg, m = self.config, self.module
        loss = torch.mean((all_ret["rgb_map"] - rgb_train) ** 2)
        total = loss
        if "rgb_map1" in all_ret:
            total = total + torch.mean((all_ret["rgb_map1"] - rgb_train) ** 2)
        if m.run_nerf and "rgb_map_nerf" in all_ret:
            total = total + torch.mean((all_ret["rgb_map_nerf"] - rgb_train) ** 2)
        if cfg.Ortho_weight > 0:
            total = total + cfg.Ortho_weight * m.density_encoding.vector_diffs() + m.rgb_encoding.vector_diffs()
        tv_on = self.tv_weight_density > 0 or self.tv_weight_app > 0
        w = None
        if tv_on:
            # the two weights decay with the learning rate; they live in a device tensor that is scaled in place, so a
            # step replayed from a CUDA graph keeps decaying them (a host float would be frozen at its recorded value)
            w = getattr(self, "_tv_weights", None)
            if w is None or w.device != loss.device:
                w = self._tv_weights = torch.tensor([self.tv_weight_density, self.tv_weight_app], device=loss.device)
            w.mul_(self.lr_factor)
        den, app = m.density_encoding, m.rgb_encoding
        if (self.l1_weight > 0 or tv_on) and den.fused_regulariser_ok() and app.fused_regulariser_ok() \
                and isinstance(self.optimizer, FusedAdam):
            # plane terms are evaluated inside the optimiser's sweep over the planes (one pass over parameters and
            # moments per step, no regulariser gradient tensor); only the few-KB lines go through autograd
            # spatial-block model parallelism: the term is the mean over the ranks' blocks (the reference gathers the
            # per-rank values and averages them, tensor_vm_encoding.py:620-636), so every rank's own planes see 1 / P
            a2a = bool(cfg.branch_parallel and cfg.get("branch_dispatch") == "a2a")
            scale = 1.0 / cfg.model_parallel_degree if cfg.branch_parallel else 1.0
            den.set_plane_regulariser(w if self.tv_weight_density > 0 else None, 0, self.l1_weight, scale)
            app.set_plane_regulariser(w if self.tv_weight_app > 0 else None, 1, 0.0, scale)
            if self.l1_weight > 0:      # in all-to-all mode the caller divides the whole objective by P afterwards
                total = total + self.l1_weight * (1.0 if a2a else scale) * den.L1_loss_lines()
        else:
            if self.l1_weight > 0:
                total = total + self.l1_weight * den.L1_loss()
            if self.tv_weight_density > 0:
                total = total + w[0] * den.TV_loss()
            if self.tv_weight_app > 0:
                total = total + w[1] * app.TV_loss()
        if getattr(self, "enable_lpips", False):
            total = total + self._lpips_term(all_ret, rgb_train)
        if self.enable_distort:
            for key in ("distort_loss", "distort_loss1", "distort_loss_nerf"):
                if key in all_ret:
                    total = total + torch.mean(all_ret[key])
        return total, loss

    def _lpips_term(self, all_ret, rgb_train):
        """``0.01 * LPIPS-VGG`` between rendered and target ``patch_size`` x ``patch_size`` patches (the batch is then made
        of whole patches; reference: benchmarks/nerf/gridnerf/gridnerf_trainer.py:271-291).  The ``lpips`` package is
        optional: without it the term is skipped with one warning."""
        net = getattr(self, "_lpips_net", None)
        if net is None:
            try:
                import lpips

                net = self._lpips_net = lpips.LPIPS(net="vgg").to(rgb_train.device)
            except Exception as exc:  # noqa: BLE001 - package or its weights are not available
                if not getattr(self, "_lpips_warned", False):
                    print(f"[{self.config.expname}] LPIPS term requested (add_lpips) but unavailable: {type(exc).__name__}: {exc}")
                    self._lpips_warned = True
                self._lpips_net = False
                return 0.0
        if net is False:
            return 0.0
        ps = int(self.config.patch_size)

        def patches(x):
            return x.reshape(-1, ps, ps, 3).permute(0, 3, 1, 2).clamp(0, 1) * 2 - 1

        target = patches(rgb_train)
        term = torch.mean(net(patches(all_ret["rgb_map"]), target))
        if self.module.run_nerf and "rgb_map_nerf" in all_ret:
            term = term + torch.mean(net(patches(all_ret["rgb_map_nerf"]), target))
        return 0.01 * term

    def train_step(self, rays_train, rgb_train, idxs_train):
        """Forward, backward, gradient sync and optimiser step on one device-resident batch.
        Returns the (detached, device) photometric MSE.  With ``cuda_graph`` the whole step is recorded
        once into a CUDA graph and replayed (one launch per step instead of a few hundred)."""
        if self._graph_ok(rays_train):
            return self._train_step_graphed(rays_train, rgb_train, idxs_train)
        return self._train_step_eager(rays_train, rgb_train, idxs_train)

    # -- whole-step CUDA graph ---------------------------------------------------------------------
    _GRAPH_WARMUP = 3

    def _graph_ok(self, rays) -> bool:
        cfg = self.config
        if not (bool(cfg.get("cuda_graph", False)) and rays.is_cuda and isinstance(self.optimizer, FusedAdam)
                and self.optimizer.capturable and self.dp_sync is None and not cfg.channel_parallel and not cfg.DDP
                and not self.timer.enabled and not getattr(self, "enable_lpips", False)):
            return False
        if cfg.branch_parallel:
            # spatial-block model parallelism is graph-safe only on the all-to-all path with kernel-path owner
            # functions (device-side row counts); every rank records and replays the same sequence of launches,
            # peer barriers and the NCCL all-reduce of the replicated heads included
            m = self.module
            return cfg.get("branch_dispatch") == "a2a" and m._use_a2a() and torch.is_grad_enabled() \
                and m._fused_app_stage_ok(rays) and m.density_encoding.fused_density_ok(rays) \
                and bool(cfg.get("fused_density", True))
        return self.mp_sync is None

    def _train_step_graphed(self, rays, rgbs, idxs):
        """Inputs are copied into fixed buffers; the first steps run eagerly (allocator and lazily built state
        settle), then one step is captured - forward, backward, deferred Adam and the schedule advance, all
        on device-resident counters - and every later call is a copy + one graph launch.  The graph is
        rebuilt when the batch shape, the sample count, the optimiser object (grid upsampling), the occupancy mask or a
        loss switch changes."""
        st = getattr(self, "_graph_state", None)
        # everything the recorded step reads from the host: a change of any of these re-records the graph
        key = (tuple(rays.shape), self.nsamples, id(self.optimizer), bool(self.module.run_nerf), bool(self.enable_distort),
               float(self.l1_weight), id(getattr(self.module, "alphaMask", None)))
        if st is None or st["key"] != key:
            st = {"key": key, "rays": torch.empty_like(rays), "rgbs": torch.empty_like(rgbs), "idxs": torch.empty_like(idxs),
                  "graph": None, "warm": 0, "loss": None}
            self._graph_state = st
        st["rays"].copy_(rays); st["rgbs"].copy_(rgbs); st["idxs"].copy_(idxs)
        if st["graph"] is None:
            if st["warm"] < self._GRAPH_WARMUP:
                st["warm"] += 1
                return self._train_step_eager(st["rays"], st["rgbs"], st["idxs"])
            torch.cuda.synchronize()
            from ...ops import native

            graph = torch.cuda.CUDAGraph()
            launches0 = native.LAUNCH_CALLS
            # thread-local: a process group's watchdog thread may touch the CUDA runtime while this thread records
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                st["loss"] = self._train_step_eager(st["rays"], st["rgbs"], st["idxs"])
            st["graph"], st["launches"] = graph, native.LAUNCH_CALLS - launches0   # library kernels recorded in the graph
            graph.replay()          # capture records without executing; the host-side counters advanced once above
            return st["loss"]
        from ...ops import native

        st["graph"].replay()
        native.LAUNCH_CALLS += st["launches"]   # the replay launches every recorded kernel again
        self.optimizer.host_advance()
        return st["loss"]

    def _train_step_eager(self, rays_train, rgb_train, idxs_train):
        cfg = self.config
        with self.timer.stage("forward"):
            rays_chunk = torch.cat((rays_train, idxs_train[:, None]), dim=-1)
            all_ret = self.model(rays_chunk, N_samples=self.nsamples)
            total, loss = self.compute_loss(all_ret, rgb_train)
            if cfg.branch_parallel and cfg.get("branch_dispatch") == "a2a":
                total = total / cfg.model_parallel_degree   # ranks hold different rays: objective is their mean
        with self.timer.stage("backward"):
            total.backward()
        with self.timer.stage("grad_sync"):
            if self.mp_sync is not None:
                self.mp_sync.sync(self._replicated_params())
            if self.dp_sync is not None:
                self.dp_sync.sync([p for g in self.optimizer.param_groups for p in g["params"]])
        with self.timer.stage("optimizer"):
            self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=True)
            owns_schedule = bool(getattr(self.optimizer, "capturable", False))   # capturable Adam decays lr on the device itself
            for group in self.optimizer.param_groups:
                if not owns_schedule:
                    group["lr"] *= self.lr_factor
                group["lr_decay"] = self.lr_factor      # lets the deferred Adam reconstruct skipped steps
        return loss.detach()

    def train(self):
        cfg = self.config
        self.model.train()
        psnrs, t0 = [], time.time()
        for self.iteration in range(cfg.start_iters, cfg.n_iters):
            it = self.iteration
            if getattr(self, "health", None) is not None:
                self.health.guard(it)      # raises PeerFailure before any kernel of this step could wait for a dead rank
            rays_train, rgb_train, idxs_train = self.data_mgr.get_rays(it)
            if cfg.add_distort > 0 and it == cfg.add_distort:
                self.enable_distort = True
            if cfg.add_lpips > 0 and it == cfg.add_lpips:
                self.enable_lpips = True               # from here on the data manager serves whole patches
                self.data_mgr.enable_lpips = True
            if cfg.add_nerf > 0 and it == cfg.add_nerf:
                self.module.run_nerf = True
                m = self.module
                lr_grid = self._group_lr(list(m.density_encoding.parameters()), cfg.lr_init)
                lr_net = self._group_lr(list(m.rgb_decoder.parameters()), cfg.lr_basis)
                self._replace_optimizer(m.get_optparam_groups(lr_grid, lr_net))
            loss = self.train_step(rays_train, rgb_train, idxs_train)
            if it % cfg.progress_refresh_rate == 0:
                mse = float(loss)
                psnrs.append(mse2psnr_npy(max(mse, 1e-10)))
                if is_main_rank():
                    print(f"[{cfg.expname}] iter {it:06d} mse {mse:.6f} psnr {psnrs[-1]:.2f} "
                          f"({(time.time() - t0) / max(it - cfg.start_iters + 1, 1) * 1e3:.1f} ms/it)", flush=True)
                    self.logger.log(it, {"Train/Loss": mse, "Train/PSNR": psnrs[-1],
                                         "Train/tf_new_lrate": self.optimizer.param_groups[0]["lr"]})
            if (it + 1) % cfg.vis_every == 0 and cfg.N_vis != 0:
                psnr_test = self.evaluation(prefix=f"{it:06d}_", n_vis=cfg.N_vis)
                self.save_ckpt()
                if is_main_rank():
                    self.logger.log(it, {"Test/PSNR": psnr_test})
                self.model.train()
            if it in cfg.update_AlphaMask_list:
                reso = self.module.gridSize.tolist()
                mask_reso = n_to_reso(min(int(np.prod(reso)), cfg.alpha_grid_reso), self.module.aabb)
                self.module.updateAlphaMask(tuple(mask_reso))
                if cfg.progressive_alpha > 0:
                    cfg.alpha_mask_filter_thre = min(cfg.alpha_mask_filter_thre + 0.1 / cfg.progressive_alpha, 0.1)
            if it in cfg.upsamp_list:
                self._upsample(self.n_voxel_list[cfg.upsamp_list.index(it)])
                self.l1_weight = cfg.L1_weight_rest
            every = int(cfg.get("async_ckpt_every", 0) or 0)
            if every > 0 and (it + 1) % every == 0:
                self.save_async(it + 1)
        if getattr(self, "_async_ckpt", None) is not None:
            self._async_ckpt.wait()
        self.save_ckpt(final=True)
        return psnrs

    # -- checkpoints -------------------------------------------------------------------------------
    def save_async(self, step: int) -> str:
        """Sharded snapshot (this rank's model and optimiser state, RNG) written off the training thread; the
        device-to-host copies run on a side stream.  Resume with ``runtime.load_sharded(latest_checkpoint(...))``."""
        from ...runtime import AsyncCheckpointer

        cfg = self.config
        if getattr(self, "_async_ckpt", None) is None:
            self._async_ckpt = AsyncCheckpointer(os.path.join(self.logfolder, "snapshots"), keep_last=2)
        for enc in (self.module.density_encoding, self.module.rgb_encoding):
            if hasattr(enc, "flush_lazy"):
                enc.flush_lazy()
        state = {"model": self.module.state_dict(), "optimizer": self.optimizer.state_dict(), "iteration": step}
        store = None
        if int(cfg.world_size) > 1:
            # the writer threads meet through the process group's rendezvous store (host side, no collective)
            from torch.distributed.distributed_c10d import _get_default_store

            store = _get_default_store()
        return self._async_ckpt.save_step(step, state, rank=int(cfg.rank), world=int(cfg.world_size), store=store,
                                          meta={"expname": cfg.expname, "model": "GridNeRF"})

    def save_ckpt(self, final: bool = False, with_optimizer: bool = True):
        """Model (and optimiser) files in the reference layout; model-parallel runs write one file per rank and, with
        ``final``, rank 0 merges them into ``state_dict-merged.th`` / ``kwargs-merged.th``."""
        cfg = self.config
        if cfg.model_parallel:
            self.module.save_model(self.logfolder, rank=cfg.mp_rank) if cfg.dp_rank == 0 else None
            if with_optimizer:
                self.save_optimizer()
            self.barrier()
            if final and cfg.rank == 0:         # spatial blocks are stacked, channel slices concatenated
                n = cfg.model_parallel_degree
                merged, kwargs = self.module.merge_ckpts(
                    [f"{self.logfolder}/state_dict-sub{r}.th" for r in range(n)],
                    [f"{self.logfolder}/kwargs-sub{r}.th" for r in range(n)])
                torch.save(merged, f"{self.logfolder}/state_dict-merged.th")
                torch.save(kwargs, f"{self.logfolder}/kwargs-merged.th")
            self.barrier()
        else:
            if is_main_rank():
                self.module.save_model(self.logfolder)
            if with_optimizer and (is_main_rank() or bool(getattr(self.optimizer, "partitioned", False))):
                self.save_optimizer()

    # -- evaluation ----------------------------------------------------------------------------------
    @torch.no_grad()
    def evaluation(self, prefix: str = "", n_vis: int = 5, save: bool = True):
        cfg = self.config
        was_train = cfg.is_train
        self.model.eval()
        test = self.data_mgr.test_dataset
        n_img = test.all_rays.shape[0]
        step = 1 if n_vis < 0 else max(n_img // n_vis, 1)
        W, H = test.img_wh
        psnrs, ssims = [], []
        dp = cfg.world_size if (cfg.DDP and not cfg.model_parallel) else 1
        for k in range(0, n_img, step):
            rays = test.all_rays[k].to(cfg.device)
            if dp > 1:  # data-parallel evaluation: each rank renders a slice of the pixels
                rays = torch.chunk(rays, dp, dim=0)[cfg.rank]
            ret = self.module.render_all_rays(rays, chunk_size=cfg.batch_size, N_samples=self.nsamples)
            rgb, depth = ret["rgb_map"].clamp(0, 1), ret["depth_map"]
            if dp > 1:
                from ...comm.varlen import all_gather_varlen

                rgb = torch.cat(all_gather_varlen(rgb), 0)
                depth = torch.cat(all_gather_varlen(depth[:, None]), 0)[:, 0]
            rgb, depth = rgb.view(H, W, 3).cpu(), depth.view(H, W).cpu()
            if test.all_rgbs is not None:
                gt = test.all_rgbs[k].view(H, W, 3)
                mse = float(torch.mean((rgb - gt) ** 2))
                psnrs.append(mse2psnr_npy(max(mse, 1e-10)))
                if cfg.get("compute_extra_metrics", False):
                    ssims.append(rgb_ssim(rgb.numpy(), gt.numpy(), 1))
            if save and is_main_rank() and not cfg.skip_save_imgs:
                depth_img, _ = visualize_depth_numpy(depth.numpy(), test.near_far)
                panel = np.concatenate(((rgb.numpy() * 255).astype(np.uint8), depth_img), axis=1)
                save_image(f"{self.logfolder}/imgs_vis/{prefix}{k:03d}.png", panel)
        cfg.is_train = was_train
        mean_psnr = float(np.mean(psnrs)) if psnrs else float("nan")
        if is_main_rank() and psnrs:
            with open(f"{self.logfolder}/imgs_vis/{prefix}mean.txt", "w", encoding="utf-8") as fh:
                fh.write(f"psnr {mean_psnr}\n" + (f"ssim {np.mean(ssims)}\n" if ssims else ""))
        return mean_psnr


def main(argv=None):
    args, unknown = get_default_parser().parse_known_args(argv)
    config = BaseConfig.from_file(args.config, parse_console_args(unknown))
    trainer = GridNeRFTrainer(config)
    trainer.train()
    psnr = trainer.evaluation(prefix="final_", n_vis=config.N_vis)
    if is_main_rank():
        print(f"final test PSNR {psnr:.3f}", flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1:])

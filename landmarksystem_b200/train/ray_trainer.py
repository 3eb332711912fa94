"""Shared trainer for the hash-grid ray models (InstantNGP, Nerfacto): sampling through the dataset
manager, log-linear learning-rate decay, gradient sync, checkpoints and evaluation (reference:
benchmarks/nerf/instant_ngp/instant_ngp_trainer.py:40-458, nerfacto/nerfacto_trainer.py:40-460)."""
from __future__ import annotations

import os
import time

import numpy as np
import torch

from ..components.data.data_manager import DatasetManager
from ..components.scene import SceneManager
from ..components.utils.image_utils import mse2psnr_npy, visualize_depth_numpy
from ..parallel.grad_sync import GradSynchronizer
from .nerf_trainer import NeRFTrainer
from .utils import is_main_rank


class RayModelTrainer(NeRFTrainer):
    model_cls = None

    def __init__(self, config):
        super().__init__(config)
        self.init_train_env()
        self.check_args()
        if not self.config.get("aabb_norm_range"):
            self.config.aabb_norm_range = [0, 1]
        self.scene_mgr = SceneManager(self.config)
        self.data_mgr = DatasetManager(self.config)
        self.iteration = config.start_iters
        self.model = self.module = self.create_model()
        self.optimizer = self.create_optimizer()
        cfg = self.config
        self.mp_sync = GradSynchronizer(cfg.mp_group, average=False) if cfg.branch_parallel else None
        if cfg.DDP and not getattr(self, "_zero_dp", False):
            self.dp_sync = GradSynchronizer(cfg.dp_group if cfg.model_parallel else None, average=True)
        else:
            self.dp_sync = None

    def create_model(self):
        cfg = self.config
        aabb = self.scene_mgr.aabb.to(cfg.device)
        self.scene_mgr.to(cfg.device)
        near_far = list(self.data_mgr.dataset_info.near_far)
        ckpt = cfg.get("ckpt")
        if ckpt == "auto":
            suffix = f"-sub{cfg.rank}" if cfg.model_parallel else ""
            ckpt = f"{self.logfolder}/state_dict{suffix}.th"
            ckpt = ckpt if os.path.exists(ckpt) else None
        model = self.model_cls(aabb, cfg.device, near_far, scene_manager=self.scene_mgr, config=cfg,
                               group=cfg.get("mp_group"))
        if ckpt:
            model.load_from_state_dict(model.get_state_dict_from_ckpt(ckpt, cfg.device), strict=False)
        return model

    def make_optimizer(self, groups):
        cfg = self.config
        on_cuda = torch.device(cfg.device).type == "cuda"
        if on_cuda and cfg.DDP and cfg.get("dp_optimizer", "p2p_zero") == "p2p_zero" and torch.distributed.is_initialized() \
                and cfg.world_size > 1:
            # data parallel on NVLink-connected GPUs: gradient reduce-scatter, partitioned Adam and parameter all-gather in
            # one peer-memory kernel per learning-rate group (the reference wraps the model in DistributedDataParallel,
            # i.e. a bucketed NCCL all-reduce of the whole hash table, benchmarks/nerf/instant_ngp/instant_ngp_trainer.py:124-125)
            from ..parallel.zero_adam import GroupedP2PZeroAdam

            self.dp_sync = None        # the fused kernel does the reduction
            self._zero_dp = True
            return GroupedP2PZeroAdam(groups, betas=(0.9, 0.999), eps=cfg.eps, group=cfg.dp_group if cfg.model_parallel else None)
        if torch.device(self.config.device).type == "cuda" and bool(self.config.get("fused_optimizer", True)):
            from ..ops import FusedAdam

            if not cfg.DDP and bool(cfg.get("hash_table_shadow", True)) and cfg.get("runtime", "Torch") == "Kernel":
                # hash tables: the backward adds into a persistent accumulator that the Adam kernel clears, and the
                # same kernel refreshes a bf16 copy that the lookup reads (half the bytes per gather; the reference's
                # tiny-cuda-nn tables are fp16 with fp32 masters).  Not under NCCL data parallelism, which averages
                # ``p.grad`` tensors.
                for mod in self.module.modules():
                    if hasattr(mod, "enable_table_shadow"):
                        mod.enable_table_shadow()
            return FusedAdam(groups, eps=self.config.eps)     # one device pass per tensor, gradients cleared in it
        return torch.optim.Adam(groups, eps=self.config.eps)

    def create_optimizer(self):
        cfg = self.config
        opt = self.optimizer = self.make_optimizer(self.module.get_optparam_groups())
        path = self._optim_path()
        if cfg.get("ckpt") and os.path.exists(path):
            opt.load_state_dict(torch.load(path, map_location=cfg.device, weights_only=False)["optimizer"])
        return opt

    def _optim_path(self):
        cfg = self.config
        per_rank = cfg.model_parallel or bool(getattr(self.optimizer, "partitioned", False))    # ZeRO shards are per rank
        suffix = f"-sub{cfg.rank}" if per_rank else ""
        return os.path.join(self.optim_dir, f"{cfg.expname}_opt{suffix}.th")

    def _replicated_params(self):
        return [p for n, p in self.module.named_parameters() if "tcnn_encoding" not in n]

    def lr_at(self, step: int) -> float:
        cfg = self.config
        t = min(step / max(cfg.lr_decay_max_steps, 1), 1.0)
        return float(np.exp(np.log(cfg.lr_init) * (1 - t) + np.log(cfg.lr_final) * t))

    def update_learning_rate(self) -> float:
        """Apply the schedule at the current iteration to every scheduled group (reference:
        instant_ngp_trainer.py:169-178)."""
        lr = self.lr_at(self.iteration)
        for group in self.optimizer.param_groups:
            if group.get("scheduled", True):
                group["lr"] = lr
        return lr

    def save_optimizer(self, path: str) -> None:
        """``{"optimizer": state_dict}`` at ``path`` (reference: instant_ngp_trainer.py:159-167)."""
        torch.save({"optimizer": self.optimizer.state_dict()}, path)

    def before_forward(self, it: int):
        pass

    def compute_loss(self, ret, rgb_train):
        return torch.mean((ret["rgb_map"] - rgb_train) ** 2)

    def train_step(self, rays_train, rgb_train, idxs_train):
        self.before_forward(self.iteration)
        rays = torch.cat((rays_train, idxs_train[:, None]), dim=-1)
        ret = self.model(rays)
        loss = self.compute_loss(ret, rgb_train)
        loss.backward()
        if self.mp_sync is not None:
            self.mp_sync.sync(self._replicated_params())
        if self.dp_sync is not None:
            self.dp_sync.sync([p for g in self.optimizer.param_groups for p in g["params"]])
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        self.update_learning_rate()
        return torch.mean((ret["rgb_map"].detach() - rgb_train) ** 2)

    def train(self):
        cfg = self.config
        self.model.train()
        t0, psnrs = time.time(), []
        for self.iteration in range(cfg.start_iters, cfg.n_iters):
            it = self.iteration
            loss = self.train_step(*self.data_mgr.get_rays(it))
            if it % cfg.progress_refresh_rate == 0:
                mse = float(loss)
                psnrs.append(mse2psnr_npy(max(mse, 1e-10)))
                if is_main_rank():
                    print(f"[{cfg.expname}] iter {it:06d} mse {mse:.6f} psnr {psnrs[-1]:.2f} "
                          f"({(time.time() - t0) / (it - cfg.start_iters + 1) * 1e3:.1f} ms/it)", flush=True)
                    self.logger.log(it, {"Train/Loss": mse, "Train/PSNR": psnrs[-1]})
            if (it + 1) % cfg.vis_every == 0 and cfg.N_vis != 0:
                ps = self.evaluation(prefix=f"{it:06d}_", n_vis=cfg.N_vis)
                self.save_ckpt()
                if is_main_rank():
                    self.logger.log(it, {"Test/PSNR": ps})
                self.model.train()
        self.save_ckpt(final=True)
        return psnrs

    def save_ckpt(self, final: bool = False):
        cfg = self.config
        os.makedirs(self.optim_dir, exist_ok=True)
        if cfg.model_parallel:
            if cfg.dp_rank == 0:
                self.module.save_model(self.logfolder, rank=cfg.mp_rank)
            self.save_optimizer(self._optim_path())
            self.barrier()
            if final and cfg.rank == 0 and cfg.branch_parallel:
                n = cfg.model_parallel_degree
                merged, kwargs = self.module.merge_ckpts([f"{self.logfolder}/state_dict-sub{r}.th" for r in range(n)],
                                                         [f"{self.logfolder}/kwargs-sub{r}.th" for r in range(n)])
                torch.save(merged, f"{self.logfolder}/state_dict-merged.th")
                torch.save(kwargs, f"{self.logfolder}/kwargs-merged.th")
            self.barrier()
        else:
            if is_main_rank():
                self.module.save_model(self.logfolder)
            if is_main_rank() or bool(getattr(self.optimizer, "partitioned", False)):
                self.save_optimizer(self._optim_path())

    @torch.no_grad()
    def evaluation(self, prefix: str = "", n_vis: int = 5, save: bool = True):
        from PIL import Image

        cfg = self.config
        self.model.eval()
        test = self.data_mgr.test_dataset
        n_img = test.all_rays.shape[0]
        step = 1 if n_vis < 0 else max(n_img // n_vis, 1)
        W, H = test.img_wh
        psnrs = []
        for k in range(0, n_img, step):
            rays = test.all_rays[k].to(cfg.device)
            ret = self.module.render_all_rays(rays, chunk_size=cfg.batch_size)
            rgb = ret["rgb_map"].clamp(0, 1).view(H, W, 3).cpu()
            depth = ret["depth_map"].view(H, W).cpu()
            if test.all_rgbs is not None:
                mse = float(torch.mean((rgb - test.all_rgbs[k].view(H, W, 3)) ** 2))
                psnrs.append(mse2psnr_npy(max(mse, 1e-10)))
            if save and is_main_rank() and not cfg.skip_save_imgs:
                dimg, _ = visualize_depth_numpy(depth.numpy(), test.near_far)
                Image.fromarray(np.concatenate(((rgb.numpy() * 255).astype(np.uint8), dimg), 1)).save(
                    f"{self.logfolder}/imgs_vis/{prefix}{k:03d}.png")
        return float(np.mean(psnrs)) if psnrs else float("nan")

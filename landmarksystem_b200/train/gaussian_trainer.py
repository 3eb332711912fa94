"""Shared training loop of the Gaussian-splatting family (vanilla / Scaffold / Octree).

Counterpart of the three nearly identical reference trainers
(benchmarks/nerf/origin_gs/gs_trainer.py:29-233, scaffold_gs/gs_trainer.py, octree_gs/gs_trainer.py):
one camera per iteration, ``0.8 L1 + 0.2 (1 - SSIM)`` (+ model-specific regulariser), densification
with optimiser-state surgery, checkpoints under ``point_cloud/iteration_N/``.
"""
from __future__ import annotations

import os
import time

import numpy as np
import torch

from ..components.data.data_manager import DatasetManager
from ..components.scene import SceneManager
from ..components.utils.image_utils import psnr
from ..components.utils.loss_utils import l1_loss, ssim
from .nerf_trainer import NeRFTrainer
from .utils import is_main_rank


class GaussianTrainerBase(NeRFTrainer):
    model_cls = None

    def __init__(self, config):
        super().__init__(config)
        self.aabb = np.array([list(config.lb), list(config.ub)], dtype=np.float32)
        self.init_train_env()
        self.check_args()
        self.scene_mgr = SceneManager(self.config)
        self.data_mgr = DatasetManager(self.config)
        self.spatial_lr_scale = float(self.data_mgr.train_dataset.cameras_extent
                                      if hasattr(self.data_mgr.train_dataset, "cameras_extent")
                                      else self.data_mgr.full_train_dataset.cameras_extent)
        self.iteration = config.start_iters
        self.model = self.create_model()
        self.optimizer = self.create_optimizer()

    def check_args(self):
        cfg = self.config
        assert not cfg.channel_parallel and not cfg.branch_parallel, "model parallelism is not defined for Gaussian models"

    # -- hooks -------------------------------------------------------------------------------------
    def build_model(self):
        raise NotImplementedError

    def extra_loss(self, image, gt_image):
        return 0.0

    def update_learning_rate(self):
        raise NotImplementedError

    def before_step(self, viewpoint_cam):
        return None

    # -- construction ----------------------------------------------------------------------------------
    def create_model(self):
        from ..components.utils.ply_utils import get_pcd

        cfg = self.config
        model = self.build_model()
        if cfg.start_checkpoint:
            state = model.get_state_dict_from_ckpt(cfg.start_checkpoint, cfg.device)
            model.load_from_state_dict(state)
        else:
            pcd = get_pcd(cfg, self.aabb, dataset=self.data_mgr.full_train_dataset)   # SfM points when the dataset has them
            model.create_from_pcd(pcd, self.spatial_lr_scale)
        return model.to(cfg.device) if hasattr(model, "to") else model

    def create_optimizer(self):
        cfg = self.config
        groups = self.model.get_optparam_groups(cfg)
        if torch.device(cfg.device).type == "cuda" and bool(cfg.get("fused_optimizer", True)):
            # one device pass per tensor with the gradient reset folded in; its state uses the keys of torch.optim.Adam
            # (``exp_avg``, ``exp_avg_sq``, ``step``), so the densification surgery on the optimiser state applies unchanged
            from ..ops import FusedAdam

            optimizer = FusedAdam(groups, lr=0.0, eps=1e-15)
        else:
            optimizer = torch.optim.Adam(groups, lr=0.0, eps=1e-15)
        if cfg.start_checkpoint:
            opt_file = os.path.join(os.path.dirname(cfg.start_checkpoint), "opt.th")
            if os.path.exists(opt_file):
                optimizer.load_state_dict(torch.load(opt_file, map_location=cfg.device, weights_only=False))
        return optimizer

    # -- loop ----------------------------------------------------------------------------------------------
    def train_step(self, viewpoint_cam, gt_image):
        cfg = self.config
        self.update_learning_rate()
        self.before_step(viewpoint_cam)
        image = self.model(viewpoint_cam)
        if image.is_cuda and image.dtype == torch.float32:
            from ..ops.ssim import fused_l1_ssim      # both terms and their gradient from one kernel each way

            Ll1, ssim_val = fused_l1_ssim(image, gt_image)
        else:
            Ll1, ssim_val = l1_loss(image, gt_image), ssim(image, gt_image)
        loss = (1.0 - cfg.lambda_dssim) * Ll1 + cfg.lambda_dssim * (1.0 - ssim_val) + self.extra_loss(image, gt_image)
        loss.backward()
        with torch.no_grad():
            self.model.densification(self.optimizer, self.iteration)
            self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=True)
        return loss.detach(), Ll1.detach(), image.detach()

    def save(self):
        folder = os.path.join(self.logfolder, "point_cloud", f"iteration_{self.iteration}")
        if is_main_rank():
            self.model.save_model(folder)
            torch.save(self.optimizer.state_dict(), os.path.join(folder, "opt.th"))
        return folder

    def train(self):
        cfg = self.config
        self.model.train()
        dev = cfg.device
        ema, t0 = 0.0, time.time()
        for self.iteration in range(cfg.start_iters + 1, cfg.n_iters + 1):
            cam, gt = self.data_mgr.get_camera("train")
            cam, gt = cam.to(dev), gt.to(dev)
            gt = gt.float() / 255.0 if cfg.img_uint8 else gt
            if self.iteration % max(self.data_mgr.train_data_size, 1) == 0 and hasattr(self.model, "oneupSHdegree"):
                self.model.oneupSHdegree()
            loss, Ll1, image = self.train_step(cam, gt)
            if self.iteration % cfg.progress_refresh_rate == 0:
                lv = float(loss)
                ema = lv if ema == 0.0 else 0.4 * lv + 0.6 * ema
                ps = float(psnr(image[None], gt[None]).mean())
                n = self.model.get_primitives_num
                if is_main_rank():
                    print(f"[{cfg.expname}] iter {self.iteration:06d} loss {ema:.5f} psnr {ps:.2f} primitives {n} "
                          f"({(time.time() - t0) / (self.iteration - cfg.start_iters) * 1e3:.1f} ms/it)", flush=True)
                    scalars = {"train_loss/l1_loss": float(Ll1), "train_loss/total_loss": lv, "train_psnr": ps,
                               "primitives_num": n}
                    if torch.device(cfg.device).type == "cuda":       # tag of the reference (origin_gs/gs_trainer.py:168-178)
                        scalars["gpu/cur_memory_allocated"] = torch.cuda.memory_allocated() / 2 ** 20
                    self.logger.log(self.iteration, scalars)
            if self.iteration in cfg.save_iterations:
                self.save()
            if self.iteration in cfg.test_iterations:
                ps = self.evaluation(os.path.join(self.logfolder, "imgs_vis"))
                if is_main_rank():
                    print(f"[ITER {self.iteration}] test PSNR {ps:.2f}", flush=True)
                    self.logger.log(self.iteration, {"Test/PSNR": ps})
                self.model.train()
        self.save()
        return self.evaluation(os.path.join(self.logfolder, "imgs_test_all"))

    @torch.no_grad()
    def evaluation(self, save_path, stride: int = None):
        from PIL import Image

        cfg = self.config
        self.model.eval()
        os.makedirs(save_path, exist_ok=True)
        n = self.data_mgr.test_data_size
        stride = stride or (20 if n >= 20 else 1)
        psnrs = []
        for idx in range(n):
            cam, gt = self.data_mgr.get_camera("test")
            if idx % stride:
                continue
            cam, gt = cam.to(cfg.device), gt.to(cfg.device)
            gt = gt.float() / 255.0 if cfg.img_uint8 else gt
            image = self.model(cam).clamp(0.0, 1.0)
            psnrs.append(float(psnr(image[None], gt[None]).mean()))
            if is_main_rank() and not cfg.skip_save_imgs:
                both = torch.cat((gt, image), dim=2).permute(1, 2, 0).cpu().numpy()
                Image.fromarray((both * 255).astype(np.uint8)).save(f"{save_path}/{idx:03d}.png")
        return float(np.mean(psnrs)) if psnrs else float("nan")

"""Evaluation engine base class (reference: landmark/train/nerf_evaluator.py:17-127) and the two
concrete evaluators shared by the model families: ray models render the test set (optionally
data-parallel over pixels), Gaussian models time every frame and report FPS."""
from __future__ import annotations

import datetime
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from ..comm import CommContext, CommMode, ParallelMode
from ..components.data.data_manager import DatasetManager
from ..components.scene import SceneManager
from ..components.utils.image_utils import mse2psnr_npy, psnr, visualize_depth_numpy
from ..components.utils.loss_utils import rgb_lpips, rgb_ssim
from ..utils import Config, EnvSetting
from .utils import is_main_rank


class NeRFEvaluator:
    def __init__(self, config):
        self.config = config
        self.model = self.data_mgr = self.scene_mgr = None
        stamp = datetime.datetime.now().strftime("-%Y%m%d-%H%M%S")
        self.logfolder = f"{config.basedir}/{config.expname}{stamp if config.add_timestamp else ''}"
        config.logfolder = self.logfolder
        self.save_folder = f"{self.logfolder}/imgs_test_all/"
        if int(os.environ.get("RANK", 0)) == 0:
            os.makedirs(self.save_folder, exist_ok=True)

    def create_model(self):
        raise NotImplementedError

    def check_args(self):
        assert self.config.get("ckpt") is not None, "Error, ckpt is None."

    def init_render_env(self):
        cfg = self.config
        torch.set_default_dtype(torch.float32)
        torch.manual_seed(cfg.random_seed)
        np.random.seed(cfg.random_seed)
        EnvSetting.refresh()
        want_cuda = torch.cuda.is_available() and str(cfg.device).startswith("cuda")
        cfg.world_size, cfg.rank = EnvSetting.WORLD_SIZE, EnvSetting.RANK
        cfg.mp_group = cfg.dp_group = None
        cfg.mp_rank = cfg.dp_rank = 0
        if cfg.world_size > 1:
            ctx = CommContext()
            if not ctx.is_initialized():
                ctx.init_distributed_env(world_size=cfg.world_size, rank=cfg.rank, backend="nccl" if want_cuda else "gloo")
                ctx.init_groups(Config(tp_size=int(cfg.channel_parallel_size or 1) if cfg.channel_parallel else 1))
            if cfg.channel_parallel:
                cfg.mp_group = ctx.get_group(ParallelMode.TENSOR_PARALLEL)
                cfg.mp_rank = ctx.get_local_rank(ParallelMode.TENSOR_PARALLEL)
            cfg.dp_group = ctx.get_group(ParallelMode.DATA_PARALLEL)
            cfg.dp_rank = ctx.get_local_rank(ParallelMode.DATA_PARALLEL) or 0
        if want_cuda:
            cfg.local_rank = EnvSetting.LOCAL_RANK % torch.cuda.device_count()
            cfg.device = torch.device("cuda", cfg.local_rank)
            torch.cuda.set_device(cfg.device)
        else:
            cfg.local_rank, cfg.device = 0, torch.device("cpu")
        tp = int(cfg.channel_parallel_size or 1) if cfg.channel_parallel else 1
        cfg.DDP = (cfg.world_size // tp) > 1
        cfg.model_parallel = bool(cfg.channel_parallel or cfg.branch_parallel)
        cfg.model_parallel_degree = tp if cfg.channel_parallel else 1

    def evaluation(self, *args, **kwargs):
        raise NotImplementedError

    @torch.no_grad()
    def eval(self):
        self.model.eval()
        psnrs = self.evaluation(self.data_mgr.test_dataset, self.config, self.save_folder, N_vis=self.config.N_vis,
                                compute_extra_metrics=self.config.get("compute_extra_metrics", False))
        mean = float(np.mean(psnrs)) if len(psnrs) else float("nan")
        if is_main_rank():
            print(f"======> {self.config.expname} test all psnr: {mean} <========================", flush=True)
        if self.config.get("render_path", False) and hasattr(self, "render_path"):
            self.render_path()
        return mean


class RayModelEvaluator(NeRFEvaluator):
    """Evaluator of GridNeRF / InstantNGP / Nerfacto: loads ``kwargs.th`` + ``state_dict.th``, optionally
    converts to channel-parallel / kernel runtime, renders the test views and writes images + ``mean.txt``."""

    model_cls = None

    def __init__(self, config):
        super().__init__(config)
        self.init_render_env()
        self.check_args()
        self.scene_mgr = SceneManager(self.config)
        self.data_mgr = DatasetManager(self.config)
        self.model = self.create_model()

    def build_from_kwargs(self, kwargs):
        return self.model_cls(**kwargs)

    def resolve_auto_ckpt(self):
        """``ckpt="auto"``: the files of the run with this ``expname`` (reference: gridnerf_evaluator.py:53-75).  A run
        without model parallelism wrote ``state_dict.th``; a model-parallel run wrote one file per rank and a merged
        one - ``ckpt_type="full"`` takes the merged file (every rank then slices what it needs), ``"sub"`` the
        file of this rank's part, which only a process that renders that part alone can use."""
        cfg = self.config
        if cfg.get("ckpt") != "auto":
            return
        if cfg.get("branch_parallel", False) or cfg.get("channel_parallel", False):
            kind = cfg.get("ckpt_type", "full")
            if kind == "full":
                suffix = "-merged"
            elif kind == "sub":
                assert int(cfg.world_size) == 1 or not cfg.get("channel_parallel", False), \
                    "ckpt_type='sub' names one rank's slice; channel-parallel rendering slices the merged file itself"
                cfg.part = int(cfg.get("part", cfg.rank) or 0)
                suffix = f"-sub{cfg.part}"
            else:
                raise ValueError(f"ckpt_type '{kind}' is not known (full, sub)")
        else:
            suffix = ""
        cfg.ckpt = f"{self.logfolder}/state_dict{suffix}.th"
        cfg.kwargs = f"{self.logfolder}/kwargs{suffix}.th"

    def create_model(self):
        from ..convertor import ComponentConvertorFactory

        cfg = self.config
        self.scene_mgr.to(cfg.device)
        self.resolve_auto_ckpt()
        kwargs_fp = cfg.get("kwargs") or cfg.ckpt.replace("state_dict", "kwargs")
        kwargs = self.model_cls.get_kwargs_from_ckpt(kwargs_fp, cfg.device)
        kwargs.update(device=cfg.device, scene_manager=self.scene_mgr, config=cfg)
        model = self.build_from_kwargs(kwargs)
        state = model.get_state_dict_from_ckpt(cfg.ckpt, cfg.device)
        model.load_from_state_dict(state, strict=False)
        if cfg.channel_parallel:
            model = ComponentConvertorFactory.get_convertor("parallelize").convert(model, cfg)
        if cfg.get("runtime", "Torch") == "Kernel":
            model = ComponentConvertorFactory.get_convertor("runtime").convert(model, cfg)
        return model.eval()

    @torch.no_grad()
    def render_path(self, savePath=None):
        """Render the ``"path"`` split (``render_path=True``: a fly-around or a trajectory file, no ground truth) into
        ``<logfolder>/imgs_path_all/``; returns the number of frames."""
        from ..components.data.datasets.dataset_utils import prep_pathdataset

        dataset = prep_pathdataset(self.config)
        savePath = savePath or f"{self.logfolder}/imgs_path_all/"
        if is_main_rank():
            os.makedirs(savePath, exist_ok=True)
        self.evaluation(dataset, self.config, savePath, N_vis=-1, prtx="path_")
        return int(dataset.all_rays.shape[0])

    def render_rays(self, rays):
        return self.model.render_all_rays(rays, chunk_size=self.config.get("render_batch_size", self.config.batch_size))

    @torch.no_grad()
    def evaluation(self, test_dataset, config, savePath=None, N_vis=5, prtx="", N_samples=-1,
                   compute_extra_metrics=False, device=None):
        from PIL import Image

        cfg = self.config
        n_img = test_dataset.all_rays.shape[0]
        step = 1 if N_vis < 0 else max(n_img // max(N_vis, 1), 1)
        W, H = test_dataset.img_wh
        dp = dist.get_world_size(cfg.dp_group) if (cfg.DDP and cfg.dp_group is not None) else 1
        psnrs, ssims, l_a, l_v, times = [], [], [], [], []
        for k in range(0, n_img, step):
            rays = test_dataset.all_rays[k].to(cfg.device)
            if cfg.device.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.time()
            if dp > 1:
                pad = (-rays.shape[0]) % dp
                if pad:
                    rays = torch.cat((rays, rays[:pad]), 0)
                part = torch.chunk(rays, dp, dim=0)[cfg.dp_rank]
                ret = self.render_rays(part)
                rgb = torch.empty(rays.shape[0], 3, device=cfg.device)
                depth = torch.empty(rays.shape[0], device=cfg.device)
                dist.all_gather_into_tensor(rgb, ret["rgb_map"].contiguous(), group=cfg.dp_group)
                dist.all_gather_into_tensor(depth, ret["depth_map"].reshape(-1).contiguous(), group=cfg.dp_group)
                rgb, depth = rgb[:H * W], depth[:H * W]
            else:
                ret = self.render_rays(rays)
                rgb, depth = ret["rgb_map"], ret["depth_map"].reshape(-1)
            if cfg.device.type == "cuda":
                torch.cuda.synchronize()
            times.append(time.time() - t0)
            rgb, depth = rgb.clamp(0, 1).view(H, W, 3).cpu(), depth.view(H, W).cpu()
            if test_dataset.all_rgbs is not None:
                gt = test_dataset.all_rgbs[k].view(H, W, 3)
                psnrs.append(mse2psnr_npy(max(float(torch.mean((rgb - gt) ** 2)), 1e-10)))
                if compute_extra_metrics:
                    ssims.append(rgb_ssim(rgb.numpy(), gt.numpy(), 1))
                    l_a.append(rgb_lpips(gt.numpy(), rgb.numpy(), "alex", cfg.device))
                    l_v.append(rgb_lpips(gt.numpy(), rgb.numpy(), "vgg", cfg.device))
            if savePath and is_main_rank() and not cfg.get("skip_save_imgs", False):
                dimg, _ = visualize_depth_numpy(depth.numpy(), test_dataset.near_far)
                Image.fromarray(np.concatenate(((rgb.numpy() * 255).astype(np.uint8), dimg), 1)).save(
                    os.path.join(savePath, f"{prtx}{k:03d}.png"))
        if is_main_rank() and times:
            lat = float(np.mean(times[1:] or times))
            print(f"average latency {lat * 1e3:.2f} ms, throughput {1.0 / lat:.2f} frames/s", flush=True)
            if savePath and psnrs:
                with open(os.path.join(savePath, f"{prtx}mean.txt"), "w", encoding="utf-8") as fh:
                    fh.write(f"psnr {np.mean(psnrs)}\n")
                    if ssims:
                        fh.write(f"ssim {np.mean(ssims)}\nlpips_alex {np.mean(l_a)}\nlpips_vgg {np.mean(l_v)}\n")
        return psnrs


class GaussianEvaluator(NeRFEvaluator):
    """Evaluator of the Gaussian family: loads ``point_cloud.ply`` (+ ``state_dict.th``), renders every
    test camera, reports PSNR, average frame time and FPS (device-synchronised wall clock per frame)."""

    model_cls = None

    def __init__(self, config):
        super().__init__(config)
        self.init_render_env()
        self.check_args()
        self.scene_mgr = SceneManager(self.config)
        self.data_mgr = DatasetManager(self.config)
        self.model = self.create_model()

    def create_model(self):
        cfg = self.config
        extent = self.data_mgr.test_dataset.cameras_extent
        model = self.model_cls(config=cfg, scene_manager=self.scene_mgr, cam_extent=extent)
        model.load_from_state_dict(model.get_state_dict_from_ckpt(cfg.ckpt, cfg.device))
        if hasattr(model, "set_appearance") and cfg.get("appearance_dim", 0) > 0:
            model.set_appearance(max(len(self.data_mgr.test_dataset), 1))
        if cfg.get("runtime", "Torch") == "Kernel" and hasattr(model, "anchor_decoder"):
            model.anchor_decoder.use_fused = True
        return model.to(cfg.device).eval()

    @torch.no_grad()
    def evaluation(self, test_dataset=None, config=None, savePath=None, N_vis=5, prtx="", N_samples=-1,
                   compute_extra_metrics=False, device=None):
        from PIL import Image

        cfg = self.config
        psnrs, times = [], []
        n = self.data_mgr.test_data_size
        step = 1 if N_vis < 0 else max(n // max(N_vis, 1), 1)
        for idx in range(n):
            cam, gt = self.data_mgr.get_camera("test")
            if idx % step:
                continue
            cam, gt = cam.to(cfg.device), gt.to(cfg.device)
            if cfg.device.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.time()
            image = self.model(cam).clamp(0.0, 1.0)
            if cfg.device.type == "cuda":
                torch.cuda.synchronize()
            times.append(time.time() - t0)
            psnrs.append(float(psnr(image[None], gt[None]).mean()))
            if savePath and is_main_rank() and not cfg.get("skip_save_imgs", False):
                both = torch.cat((gt, image), dim=2).permute(1, 2, 0).cpu().numpy()
                Image.fromarray((both * 255).astype(np.uint8)).save(os.path.join(savePath, f"{prtx}{idx:03d}.png"))
        if is_main_rank() and times:
            lat = float(np.mean(times[1:] or times))
            print(f"average time {lat * 1e3:.2f} ms, FPS {1.0 / lat:.2f}, primitives {self.model.get_primitives_num}", flush=True)
        return psnrs


def evaluator_main(evaluator_cls, argv=None):
    """Shared command-line entry of the six model evaluators: ``--config <render conf.py> [--key value ...]``."""
    from ..configs import BaseConfig, get_default_parser, parse_console_args

    args, unknown = get_default_parser().parse_known_args(argv)
    config = BaseConfig.from_file(args.config, parse_console_args(unknown))
    config.is_train = False
    return evaluator_cls(config).eval()

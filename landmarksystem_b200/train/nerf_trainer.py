"""Training engine base class (reference: landmark/train/nerf_trainer.py:25-277).

Owns the log-folder layout, seeding, distributed bootstrap and parallel-group algebra; concrete
trainers implement ``create_model / create_optimizer / train / evaluation``.
"""
from __future__ import annotations

import datetime
import os
import random
import shutil

import numpy as np
import torch
import torch.distributed as dist

from ..comm import CommContext, CommMode, init_train_groups
from ..comm.train_groups import mp_degree_of
from ..components.utils.system_utils import set_print_with_timestamp
from ..utils import EnvSetting
from ..utils.metrics import MetricsLogger, StageTimer
from .utils import is_main_rank


class NeRFTrainer:
    def __init__(self, config):
        self.config = config
        self.device = config.device
        self.model = self.module = self.optimizer = self.data_mgr = self.scene_mgr = None
        self.metrics = {}
        stamp = datetime.datetime.now().strftime("-%Y%m%d-%H%M%S")
        self.logfolder = f"{config.basedir}/{config.expname}{stamp if config.add_timestamp else ''}"
        config.logfolder = self.logfolder
        self.optim_dir = config.optim_dir if config.get("optim_dir") is not None else self.logfolder + "/optim/"
        self.save_folder = f"{self.logfolder}/imgs_test_all/"
        self.writer = None
        main = int(os.environ.get("RANK", 0)) == 0
        if main:
            for d in (self.logfolder, f"{self.logfolder}/imgs_vis", self.optim_dir, self.save_folder):
                os.makedirs(d, exist_ok=True)
            config.save_config(os.path.join(self.logfolder, f"args-{stamp}.txt"))
            src = config.get("config")
            if src and os.path.exists(str(src)):
                shutil.copyfile(str(src), os.path.join(self.logfolder, "config.txt"))
        self.logger = MetricsLogger(self.logfolder if main else None, tensorboard=bool(config.get("tensorboard")),
                                    wandb=bool(config.get("wandb")), run_name=str(config.get("expname")),
                                    run_config={k: v for k, v in dict(config).items() if isinstance(v, (int, float, str, bool, list))})
        self.writer = self.logger.writer
        self.timer = StageTimer(enabled=bool(config.get("profile", False)))

    # -- environment ------------------------------------------------------------------
    def init_train_env(self):
        cfg = self.config
        torch.set_default_dtype(torch.float32)
        torch.manual_seed(cfg.random_seed)
        np.random.seed(cfg.random_seed)
        random.seed(cfg.random_seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(cfg.random_seed)
        torch.backends.cudnn.deterministic = True
        if cfg.get("print_timestamp", False):
            set_print_with_timestamp()
        EnvSetting.refresh()
        want_cuda = torch.cuda.is_available() and str(cfg.device).startswith("cuda")
        if EnvSetting.WORLD_SIZE > 1 or "MASTER_ADDR" in os.environ:
            ctx = CommContext()
            if not ctx.is_initialized():
                ctx.init_distributed_env(world_size=EnvSetting.WORLD_SIZE, rank=EnvSetting.RANK,
                                         backend="nccl" if want_cuda else "gloo", timeout=EnvSetting.COMM_TIMEOUT)
            cfg.rank, cfg.world_size = ctx.get_global_rank(), ctx.get_world_size(CommMode.GLOBAL)
        else:
            cfg.rank, cfg.world_size = 0, 1
        # failure detection: heartbeats through the job's key-value store, checked between steps
        self.health = None
        if cfg.get("heartbeat", False) and cfg.world_size > 1 and torch.distributed.is_initialized():
            from ..runtime import HeartbeatMonitor

            store = torch.distributed.distributed_c10d._get_default_store()
            self.health = HeartbeatMonitor(store, cfg.rank, cfg.world_size, timeout=float(cfg.get("heartbeat_timeout", 30.0))).start()
        if want_cuda:
            cfg.local_rank = EnvSetting.LOCAL_RANK % torch.cuda.device_count()
            cfg.device = torch.device("cuda", cfg.local_rank)
            torch.cuda.set_device(cfg.device)
        else:
            cfg.local_rank, cfg.device = 0, torch.device("cpu")
        self.device = cfg.device
        cfg.model_parallel = bool(cfg.channel_parallel or cfg.branch_parallel)
        cfg.model_parallel_degree = mp_degree_of(cfg)
        init_train_groups(cfg)
        if not cfg.model_parallel and cfg.world_size > 1:
            assert cfg.DDP, "world size > 1 without model parallelism requires DDP=True"

    def check_args(self):
        cfg = self.config
        assert sum([bool(cfg.channel_parallel), bool(cfg.branch_parallel)]) <= 1, \
            "only one of channel / branch parallel can be enabled"
        mp = cfg.model_parallel_degree if cfg.model_parallel else 1
        if cfg.DDP:
            assert cfg.world_size % mp == 0 and cfg.world_size >= mp, \
                f"world size ({cfg.world_size}) must be a multiple of the model-parallel size ({mp}) with DDP"
        else:
            assert cfg.world_size == mp, f"world size ({cfg.world_size}) must equal the model-parallel size ({mp})"

    # -- to be provided by concrete trainers --------------------------------------------------
    def create_model(self):
        raise NotImplementedError

    def create_optimizer(self):
        raise NotImplementedError

    def train(self, *args, **kwargs):
        raise NotImplementedError

    def evaluation(self, *args, **kwargs):
        raise NotImplementedError

    @torch.no_grad()
    def eval(self) -> float:
        """Evaluate the current model on the test split and return the mean PSNR (reference:
        landmark/train/nerf_trainer.py:208-300).  Ray trainers write ``<logfolder>/imgs_vis/test_all_*``, camera
        trainers ``<logfolder>/imgs_test_all/*``."""
        import inspect

        self.model.eval()
        params = inspect.signature(self.evaluation).parameters
        if "save_path" in params:
            value = self.evaluation(os.path.join(self.logfolder, "imgs_test_all"))
        else:
            value = self.evaluation(prefix="test_all_", n_vis=int(self.config.get("N_vis", -1)))
        if dist.is_initialized() and dist.get_rank() != 0:
            return value
        print(f"======> {self.config.expname} test all psnr: {value} <========================", flush=True)
        return value

    def barrier(self):
        if dist.is_initialized():
            dist.barrier()

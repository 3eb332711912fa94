"""Training switches shared by every model family
(reference: landmark/nerf_components/configs/train_config.py:9-91)."""
from typing import List, Optional, Union

import torch
from typing_extensions import Literal

from .base_configclass import ConfigClass


class TrainConfig(ConfigClass):
    model_name: str
    expname: str
    start_iters: int = 0
    n_iters: int
    batch_size: int = 4096
    progress_refresh_rate: int = 10
    wandb: bool = False
    tensorboard: bool = False
    basedir: str = "./log"
    add_timestamp: bool = False
    random_seed: int = 20211202
    debug: bool = False
    N_vis: int = 5
    vis_every: int = 10000
    skip_save_imgs: bool = False
    optim_dir: Optional[str] = None
    ckpt: Optional[str] = None
    ckpt_type: Literal["full", "sub"] = "full"
    kwargs: Optional[str] = None

    is_train: bool = True
    device: Union[str, torch.device] = torch.device("cuda")

    # parallel switches
    DDP: bool = False
    channel_parallel: bool = False
    branch_parallel: bool = False
    plane_division: Optional[list] = [1, 1]
    channel_parallel_size: Optional[int] = None
    model_parallel_and_DDP: bool = False

    # Gaussian-family schedule
    test_iterations: List[int] = []
    save_iterations: List[int] = []
    start_checkpoint: Optional[str] = None

    print_timestamp: bool = True

    # additions of this framework
    dp_optimizer: Literal["p2p_zero", "nccl_allreduce"] = "p2p_zero"   # data-parallel gradient path on GPUs
    heartbeat: bool = False      # multi-rank failure detection: heartbeats in the rendezvous store, checked every step
    heartbeat_timeout: float = 30.0
    async_ckpt_every: int = 0    # > 0: sharded asynchronous snapshot every N iterations (log dir / snapshots)
    cuda_graph: bool = False     # record the whole training step once in a CUDA graph and replay it (single-GPU fused path)
    profile: bool = False                                              # CUDA-event stage timers + NVTX ranges

    def check_args(self) -> None:
        super().check_args()
        if self.plane_division is not None:
            assert len(self.plane_division) == 2, "plane_division is [nx, ny]"
        assert not (self.channel_parallel and self.branch_parallel), "enable one model-parallel mode at a time"

"""Rendering switches (reference: landmark/nerf_components/configs/render_config.py:10-92)."""
from typing import List, Optional, Union

import torch
from typing_extensions import Literal

from .base_configclass import ConfigClass
from .train_config import TrainConfig

_INHERITED = ("model_name", "expname", "basedir", "add_timestamp", "random_seed", "debug", "N_vis", "device",
              "plane_division")


class RenderConfig(ConfigClass):
    model_name: Optional[str] = None
    expname: Optional[str] = None
    batch_size: int = 4096
    basedir: str = "./log"
    add_timestamp: bool = False
    random_seed: int = 20211202
    debug: bool = False
    N_vis: int = 5
    ckpt: Optional[str] = None
    ckpt_type: Literal["full", "sub"] = "full"
    kwargs: Optional[str] = None
    is_train: bool = False
    distributed: bool = False
    device: Union[str, torch.device] = torch.device("cuda")
    DDP: bool = False
    channel_parallel: bool = False
    branch_parallel: bool = False
    plane_division: Optional[list] = None
    channel_parallel_size: Optional[int] = None
    model_parallel_and_DDP: bool = False
    test_iterations: List[int] = []
    save_iterations: List[int] = []
    quiet: bool = False
    start_checkpoint: Optional[str] = None
    compute_extra_metrics: bool = False

    def from_train_config(self, train_config: TrainConfig) -> "RenderConfig":
        """Fill every unset (``None``) inheritable field from ``train_config``."""
        for name in _INHERITED:
            if getattr(self, name, None) is None and hasattr(train_config, name):
                setattr(self, name, getattr(train_config, name))
        return self

    def check_args(self) -> None:
        super().check_args()
        assert not self.is_train, "RenderConfig is not for training"

"""Dataset description (reference: landmark/nerf_components/configs/dataset_config.py:8-86)."""
from typing import List, Optional, Union

import torch
from typing_extensions import Literal

from .base_configclass import ConfigClass


def _is_vec3(value) -> bool:
    if isinstance(value, torch.Tensor):
        return tuple(value.shape) == (3,)
    return isinstance(value, (list, tuple)) and len(value) == 3


class DatasetConfig(ConfigClass):
    partition: str = "all"
    datadir: str
    subfolder: Optional[list] = None
    dataset_name: Literal["city", "matrixcity", "blender", "Colmap", "colmap", "zhangjiang", "synthetic"] = "city"
    dataset_type: Literal["nerf", "gaussian"] = "nerf"
    use_preprocessed_data: bool = False
    processed_data_type: str = "file"
    preprocessed_dir: str = "./preprocessed_data/"
    downsample_train: int = 1
    train_all_data: bool = False
    img_uint8: bool = False
    preload: bool = False
    dynamic_load: bool = False
    max_iter_each_block: int = -1
    lb: Union[List[float], torch.Tensor] = [0, 0, 0]
    ub: Union[List[float], torch.Tensor] = [0, 0, 0]
    pose_rotation: Union[List[float], torch.Tensor] = [0, 0, 0]
    pose_translation: Union[List[float], torch.Tensor] = [0, 0, 0]

    def check_args(self) -> None:
        super().check_args()
        assert not self.dynamic_load or self.dataset_type == "gaussian", \
            "dynamic_load is only supported for gaussian datasets"
        assert not self.use_preprocessed_data or self.dataset_type == "nerf", \
            "use_preprocessed_data is only supported for nerf datasets"
        for name in ("lb", "ub", "pose_rotation", "pose_translation"):
            assert _is_vec3(getattr(self, name)), f"{name} must have 3 components"

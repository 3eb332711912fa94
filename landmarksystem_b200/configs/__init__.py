from .base_configclass import ConfigClass
from .config_parser import BaseConfig, get_default_parser, parse_console_args
from .dataset_config import DatasetConfig
from .render_config import RenderConfig
from .train_config import TrainConfig

__all__ = ["ConfigClass", "BaseConfig", "get_default_parser", "parse_console_args", "DatasetConfig",
           "RenderConfig", "TrainConfig"]

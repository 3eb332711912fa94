"""Typed configuration blocks (``TrainConfig`` / ``RenderConfig``, ``DatasetConfig``, one block per model family) and the
loader that flattens a configuration file's blocks into one namespace (``BaseConfig.from_file``)."""
from . import base_configclass as _blocks
from . import config_parser as _parser
from . import dataset_config as _dataset
from . import render_config as _render
from . import train_config as _train

ConfigClass = _blocks.ConfigClass
TrainConfig, RenderConfig, DatasetConfig = _train.TrainConfig, _render.RenderConfig, _dataset.DatasetConfig
BaseConfig = _parser.BaseConfig
get_default_parser, parse_console_args = _parser.get_default_parser, _parser.parse_console_args

__all__ = ["BaseConfig", "ConfigClass", "DatasetConfig", "RenderConfig", "TrainConfig", "get_default_parser",
           "parse_console_args"]

"""Framework-wide utilities and string constants (reference: landmark/utils/__init__.py:6-11)."""
from .config import Config
from .env import EnvSetting, parse_env
from .singleton import SingletonMeta

_RANK_STR = "rank"
_WORLD_SIZE_STR = "world_size"
_PARALLEL_CONFIG_STR = "parallel_config"
_OFFLOAD_CONFIG_STR = "offload_config"
MERGE_TYPE_STR = "merge_type"

__all__ = [
    "Config",
    "EnvSetting",
    "parse_env",
    "SingletonMeta",
    "_RANK_STR",
    "_WORLD_SIZE_STR",
    "_PARALLEL_CONFIG_STR",
    "_OFFLOAD_CONFIG_STR",
    "MERGE_TYPE_STR",
]

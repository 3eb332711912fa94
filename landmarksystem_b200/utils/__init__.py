"""Framework-wide utilities: attribute-access configuration dictionary, launcher environment, singleton metaclass and
the key names of the inference configuration (reference: landmark/utils/__init__.py:6-11)."""
from .config import Config
from .constants import _OFFLOAD_CONFIG_STR, _PARALLEL_CONFIG_STR, _RANK_STR, _WORLD_SIZE_STR, MERGE_TYPE_STR
from .env import EnvSetting, parse_env
from .singleton import SingletonMeta

__all__ = ["Config", "EnvSetting", "SingletonMeta", "parse_env", "MERGE_TYPE_STR", "_OFFLOAD_CONFIG_STR",
           "_PARALLEL_CONFIG_STR", "_RANK_STR", "_WORLD_SIZE_STR"]

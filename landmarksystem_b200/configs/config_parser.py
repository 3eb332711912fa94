"""Config-file loader and console override parser
(reference: landmark/nerf_components/configs/config_parser.py:9-156).

A conf file is a Python file that defines ``config = [blockA, blockB, ...]`` where each
block is a :class:`ConfigClass`.  All blocks are validated and flattened into one
namespace; ``--key value`` console pairs may override int/float/str/bool entries.
"""
from __future__ import annotations

import argparse
import runpy
import sys
from pathlib import Path
from typing import Dict, Iterable, Optional

from ..utils.config import Config

_SCALARS = (int, float, str, bool)
_TRUE, _FALSE = {"true", "1", "yes"}, {"false", "0", "no"}


def get_default_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser()
    parser.add_argument("--config", type=str, help="path to the config file")
    return parser


def parse_console_args(unknown_args: Optional[Iterable[str]]) -> Optional[Dict[str, object]]:
    """Turn ``["--a", "1", "--flag", "--b", "x"]`` into ``{"a": "1", "flag": True, "b": "x"}``."""
    if unknown_args is None:
        return None
    tokens = list(unknown_args)
    parsed: Dict[str, object] = {}
    pos = 0
    while pos < len(tokens):
        token = tokens[pos]
        pos += 1
        if not token.startswith("--"):
            continue
        if pos < len(tokens) and not tokens[pos].startswith("--"):
            parsed[token[2:]] = tokens[pos]
            pos += 1
        else:
            parsed[token[2:]] = True
    return parsed


def _coerce(name: str, raw, target_type):
    if target_type is bool:
        if isinstance(raw, bool):
            return raw
        low = str(raw).lower()
        if low in _TRUE:
            return True
        if low in _FALSE:
            return False
        raise ValueError(f"Unknown boolean value {raw} for argument {name}.")
    try:
        return target_type(raw)
    except Exception as exc:
        raise ValueError(f"Invalid value {raw} for argument {name}.") from exc


def _from_text(raw):
    if not isinstance(raw, str):
        return raw
    low = raw.lower()
    if low in ("none", "null"):
        return None
    if low in ("true", "false"):
        return low == "true"
    for kind in (int, float):
        try:
            return kind(raw)
        except ValueError:
            pass
    return raw


class BaseConfig(Config):
    """Flattened run configuration."""

    @staticmethod
    def from_file(filename, console_args=None, merge_configs: bool = True) -> "BaseConfig":
        path = Path(filename).absolute()
        assert path.exists(), f"{filename} is not found, please check your configuration path"
        assert path.suffix == ".py", "only .py files are supported"

        added = str(path.parent) not in sys.path
        if added:  # lets `from other_conf import *` resolve siblings
            sys.path.insert(0, str(path.parent))
        try:
            namespace = runpy.run_path(str(path))
        finally:
            if added:
                sys.path.remove(str(path.parent))
        assert "config" in namespace, f"{filename} does not have config attribute"

        cfg = BaseConfig()
        cfg["config"] = str(filename)
        for block in namespace["config"]:
            block.check_args()
            if merge_configs:
                for key, value in block:
                    assert key not in cfg, f"Duplicate attribute {key} in configs."
                    cfg._add_item(key, value)
            else:
                cfg._add_item(type(block).__name__, block)

        for key, raw in (console_args or {}).items():
            assert key in cfg, f"Unknown argument {key}."
            target = type(cfg[key])
            if target.__name__ == "device":  # torch.device given as a string on the console
                import torch

                cfg[key] = torch.device(str(raw))
                continue
            if cfg[key] is None:
                # a field that is unset in the file (``ckpt``, ``kwargs``, ``point_path``, ...) carries no type to coerce
                # to: take the text as it stands, with the usual spellings of none / numbers / booleans recognised
                cfg[key] = _from_text(raw)
                continue
            assert target in _SCALARS, \
                f"Unsupported type {target} for argument {key}, please set this argument in config file."
            cfg[key] = _coerce(key, raw, target)
        return cfg

    def _add_item(self, key, value):  # keep pydantic blocks / plain dicts untouched
        dict.__setitem__(self, key, value)

    def save_config(self, file_path: str) -> None:
        with open(file_path, "w", encoding="utf-8") as handle:
            for key in sorted(self):
                handle.write(f"{key} = {self[key]}\n")

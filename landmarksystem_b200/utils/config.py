"""Attribute-style configuration dictionary.

Behavioural counterpart of the reference's ``Config`` (landmark/utils/config.py:7-95):
a ``dict`` whose keys are also attributes, nested dicts become nested ``Config``
objects, and ``from_file`` evaluates a ``.py`` file and keeps its plain globals.
"""
from __future__ import annotations

import inspect
import runpy
from pathlib import Path
from typing import Any, Mapping


class Config(dict):
    """``dict`` with attribute access; nested mappings are wrapped recursively."""

    def __init__(self, mapping: Mapping[str, Any] | None = None, **kwargs: Any):
        super().__init__()
        merged = dict(mapping or {})
        merged.update(kwargs)
        for key, value in merged.items():
            self._add_item(key, value)

    # -- attribute protocol -------------------------------------------------
    def __getattr__(self, key: str) -> Any:
        try:
            return self[key]
        except KeyError as exc:  # keeps hasattr()/getattr(default) working
            raise AttributeError(key) from exc

    def __setattr__(self, key: str, value: Any) -> None:
        self._add_item(key, value)

    def __delattr__(self, key: str) -> None:
        try:
            del self[key]
        except KeyError as exc:
            raise AttributeError(key) from exc

    def __missing__(self, key: str) -> Any:
        raise KeyError(key)

    def _add_item(self, key: str, value: Any) -> None:
        if isinstance(value, Mapping) and not isinstance(value, Config):
            value = Config(value)
        dict.__setitem__(self, key, value)

    def update(self, other: Mapping[str, Any] | None = None, **kwargs: Any) -> "Config":  # type: ignore[override]
        merged = dict(other or {})
        merged.update(kwargs)
        for key, value in merged.items():
            self._add_item(key, value)
        return self

    def to_dict(self) -> dict:
        out = {}
        for key, value in self.items():
            out[key] = value.to_dict() if isinstance(value, Config) else value
        return out

    # -- file loading -------------------------------------------------------
    @staticmethod
    def from_file(filename: str | Path) -> "Config":
        """Run ``filename`` (a ``.py`` file) and collect its data globals."""
        path = Path(filename).absolute()
        if not path.exists():
            raise FileNotFoundError(f"{filename} is not found, please check your configuration path")
        if path.suffix != ".py":
            raise ValueError("only .py files are supported")
        namespace = runpy.run_path(str(path))
        cfg = Config()
        for key, value in namespace.items():
            if key.startswith("__") or inspect.ismodule(value) or inspect.isclass(value):
                continue
            cfg._add_item(key, value)
        return cfg

"""Common base of every model and component (reference:
landmark/nerf_components/model/base_module.py:8-113).

Two services: (1) ``merge_config`` - for each parameter name, along which dimension spatial blocks
are stacked (used by checkpoint merge/split and by dynamic loading); (2) constructor-argument
capture so that a convertor can re-instantiate a component as its parallel or fused subclass.
"""
from __future__ import annotations

import inspect
from typing import Any, Dict, Mapping

from torch import nn


class BaseModule(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.merge_config: Dict[str, Any] = {}
        self._init_kwargs: Dict[str, Any] = {}

    # -- merge configuration ----------------------------------------------------
    def get_merge_config(self, prefix: str = "") -> Dict[str, Any]:
        merged = dict(getattr(self, "merge_config", {}) or {})
        for name, child in self.named_children():
            if isinstance(child, BaseModule):
                for key, value in child.get_merge_config().items():
                    merged[f"{prefix}{name}.{key}"] = value
        return merged

    def set_merge_config(self, merge_config: Mapping[str, Any]) -> None:
        for name, child in self.named_children():
            if isinstance(child, BaseModule):
                head = name + "."
                child.set_merge_config({k[len(head):]: v for k, v in merge_config.items() if k.startswith(head)})
        for key, value in merge_config.items():
            if key in self.merge_config:
                self.merge_config[key] = value

    # -- constructor capture ------------------------------------------------------
    def save_init_kwargs(self, local_dict: Mapping[str, Any]) -> None:
        init = type(self).__init__
        init = getattr(init, "_origin_init", init)
        names = list(inspect.signature(init).parameters)[1:]
        self._init_kwargs = {n: local_dict[n] for n in names if n in local_dict}

    def get_init_kwargs(self) -> Dict[str, Any]:
        return dict(self._init_kwargs)

    # -- checkpoint protocol (overridden by models) -------------------------------------
    @staticmethod
    def get_kwargs() -> Mapping[str, Any]:
        raise NotImplementedError

    @staticmethod
    def get_kwargs_from_ckpt(file_path, map_location) -> Mapping[str, Any]:
        raise NotImplementedError

    def get_state_dict_from_ckpt(self, file_path, map_location, prefix: str = "") -> Mapping[str, Any]:
        raise NotImplementedError

    def load_from_state_dict(self, state_dict: Mapping[str, Any], strict: bool = True):
        raise NotImplementedError

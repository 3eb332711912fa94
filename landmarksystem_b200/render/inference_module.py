"""User-facing inference adapters (reference: landmark/render/util/inference_module.py:12-163).
An ``InferenceModule`` wraps a model and defines ``preprocess`` (user arguments -> model inputs),
``forward`` and ``postprocess`` (model outputs -> what the caller receives)."""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

from torch import nn

from ..components.scene import SceneManager


class InferenceInterface(nn.Module):
    def preprocess(self, *args, **kwargs):
        return args, kwargs

    def postprocess(self, *args, **kwargs):
        if len(args) == 1 and not kwargs:
            return args[0]
        return args if not kwargs else (args, kwargs)


class InferenceModule(InferenceInterface):
    def __init__(self, model: Optional[nn.Module] = None) -> None:
        super().__init__()
        self.model = model
        self.scene_mgr = None

    @property
    def inter_model(self):
        return self.model

    @inter_model.setter
    def inter_model(self, model):
        self.model = model

    @property
    def scene_manager(self):
        if self.scene_mgr is None and self.model is not None:
            for value in vars(self.model).values():
                if isinstance(value, SceneManager):
                    self.scene_mgr = value
        return self.scene_mgr

    @property
    def merge_config(self):
        return self.model.get_merge_config()

    def get_merge_config(self):
        return self.model.get_merge_config()

    def channel_last(self):
        self.model.channel_last()

    def get_state_dict_from_ckpt(self, file_path, map_location) -> Mapping[str, Any]:
        return self.model.get_state_dict_from_ckpt(file_path, map_location)

    def load_from_state_dict(self, state_dict: Mapping[str, Any], strict: bool = False):
        return self.model.load_from_state_dict(state_dict, strict)

    def preprocess(self, *args, **kwargs):
        if self.model is not None and hasattr(self.model, "preprocess"):
            return self.model.preprocess(*args, **kwargs)
        return super().preprocess(*args, **kwargs)

    def postprocess(self, *args, **kwargs):
        if self.model is not None and hasattr(self.model, "postprocess"):
            return self.model.postprocess(*args, **kwargs)
        return super().postprocess(*args, **kwargs)

    def forward(self, *args, **kwargs):
        assert self.model is not None
        return self.model(*args, **kwargs)

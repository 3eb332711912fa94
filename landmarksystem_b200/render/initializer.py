"""Builds the inference model from a checkpoint's kwargs + the model config (reference:
landmark/render/util/initializer.py:6-44).  Models are constructed on the CPU; the engine moves them."""
from __future__ import annotations

import inspect

from ..components.model.base_model import BaseGaussian, BaseNeRF
from ..components.scene import SceneManager
from ..utils import _OFFLOAD_CONFIG_STR


class InferenceModuleInitializer:
    def __init__(self, based_model_cls, infer_model_cls):
        self.based_model_cls, self.infer_model_cls = based_model_cls, infer_model_cls

    def get_infer_model(self, model_config, inference_config):
        if model_config is None:
            kwargs = self.based_model_cls.get_kwargs()
        else:
            assert model_config.get("ckpt") is not None, "should set the checkpoint file path"
            if inference_config.get("ckpt_path") is not None:
                assert inference_config.ckpt_path == model_config.ckpt
            else:
                inference_config.ckpt_path = model_config.ckpt
            kwargs = {}
            if model_config.get("kwargs") is not None:
                kwargs = self.based_model_cls.get_kwargs_from_ckpt(model_config.kwargs, "cpu")
            kwargs["config"] = model_config
            if _OFFLOAD_CONFIG_STR in inference_config and issubclass(self.based_model_cls, BaseGaussian):
                raise AssertionError("not support offload in Gaussian models")
            model_config.device = "cpu"
            model_config.grids_come_from_ckpt = True      # the engine loads the checkpoint right after construction
            kwargs["scene_manager"] = SceneManager(model_config)
            if "device" in kwargs:
                kwargs["device"] = "cpu"
        assert issubclass(self.based_model_cls, (BaseNeRF, BaseGaussian)), \
            f"Unknown support model type {self.based_model_cls}"
        cls = self.infer_model_cls if self.infer_model_cls is not None else self.based_model_cls
        accepted = inspect.signature(cls.__init__).parameters
        if not any(p.kind == inspect.Parameter.VAR_KEYWORD for p in accepted.values()):
            kwargs = {k: v for k, v in kwargs.items() if k in accepted}
        return cls(**kwargs)

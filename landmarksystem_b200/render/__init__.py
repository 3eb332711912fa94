"""Rendering (inference) engine.  Heavy submodules are imported on first attribute access so that
``landmarksystem_b200.render.types`` can be used by the component layer without import cycles."""
from .types import MergeType, RuntimeType, StageInput


__all__ = ["InferenceEngine", "InferenceInterface", "InferenceModule", "InferenceModuleInitializer", "MergeType",
           "RuntimeType", "StageInput", "transform_gridnerf_model_to_channel_last", "transform_gs_mlp_checkpoint"]

# names the reference exports from ``landmark.render`` and ``landmark.render.util`` -> the module that defines them
_LAZY = {"InferenceEngine": "inference_engine", "InferenceInterface": "inference_module",
         "InferenceModule": "inference_module", "InferenceModuleInitializer": "initializer",
         "transform_gridnerf_model_to_channel_last": "utils", "transform_gs_mlp_checkpoint": "utils"}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        return getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
    raise AttributeError(name)

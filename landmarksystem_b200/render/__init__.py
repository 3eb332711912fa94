"""Rendering (inference) engine.  Heavy submodules are imported on first attribute access so that
``landmarksystem_b200.render.types`` can be used by the component layer without import cycles."""
from .types import MergeType, RuntimeType

__all__ = ["InferenceEngine", "InferenceInterface", "InferenceModule", "MergeType", "RuntimeType"]


def __getattr__(name):
    if name == "InferenceEngine":
        from .inference_engine import InferenceEngine

        return InferenceEngine
    if name in ("InferenceInterface", "InferenceModule"):
        from . import inference_module

        return getattr(inference_module, name)
    raise AttributeError(name)

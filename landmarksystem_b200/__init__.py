"""landmarksystem_b200: a B200-native large-scene reconstruction framework (GridNeRF, InstantNGP,
Nerfacto, vanilla / Scaffold / Octree 3D Gaussian splatting) with training and rendering engines.

Public entry points mirror the reference package (landmark/__init__.py:22-99):
``init_inference(model_cls, infer_cls, model_config, inference_config) -> InferenceEngine``.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Union

from .utils import Config, EnvSetting, _OFFLOAD_CONFIG_STR, _PARALLEL_CONFIG_STR, _RANK_STR, _WORLD_SIZE_STR

__version__ = "0.1.0"


def _transform_to_cls(config: Union[str, Path, Config, Dict]) -> Config:
    if isinstance(config, (str, Path)):
        return Config.from_file(config)
    if not isinstance(config, Config) and isinstance(config, dict):
        return Config(config)
    return config


def _update_global_info(parallel_config) -> Config:
    EnvSetting.refresh()
    parallel_config = Config(parallel_config)
    parallel_config[_RANK_STR] = EnvSetting.RANK
    parallel_config[_WORLD_SIZE_STR] = EnvSetting.WORLD_SIZE
    return parallel_config


def _launch(parallel_config) -> Config:
    from .comm import init_communication_context

    parallel_config = _update_global_info(parallel_config)
    init_communication_context(parallel_config)
    return parallel_config


def _infer_config_sanity_check(model_config, inference_config) -> None:
    if model_config is not None and model_config.get("act_cache") and inference_config.get(_OFFLOAD_CONFIG_STR) is not None:
        raise AssertionError("Offload is not supported when act_cache is True")
    if inference_config.get(_OFFLOAD_CONFIG_STR) is not None and inference_config.get(_PARALLEL_CONFIG_STR) is not None:
        assert not int(inference_config[_PARALLEL_CONFIG_STR].get("tp_size", 1)) > 1, \
            "Offload is not supported when tp_size > 1, please set tp_size to 1 or disable tensor parallel"
    assert not inference_config.get("half_precision", False), "Half precision is not supported yet"
    assert not inference_config.get("static_allocation", False), "Static allocation is not supported yet"


def init_inference(based_model_cls, infer_model_cls, model_config, inference_config):
    """Build an :class:`~landmarksystem_b200.render.InferenceEngine` for ``based_model_cls`` wrapped by
    ``infer_model_cls`` (an ``InferenceModule`` subclass that defines pre/post-processing)."""
    from .render.inference_engine import InferenceEngine
    from .render.initializer import InferenceModuleInitializer

    inference_config = _transform_to_cls(inference_config)
    model_config = _transform_to_cls(model_config)
    if inference_config.get(_PARALLEL_CONFIG_STR) is not None:
        inference_config[_PARALLEL_CONFIG_STR] = _launch(inference_config[_PARALLEL_CONFIG_STR])
    _infer_config_sanity_check(model_config, inference_config)
    model = InferenceModuleInitializer(based_model_cls, infer_model_cls).get_infer_model(model_config, inference_config)
    return InferenceEngine(model, inference_config)


def init_training(trainer_cls, config):
    """Construct a trainer from a flattened run configuration (the reference leaves this entry point
    unimplemented, landmark/__init__.py:95-96)."""
    return trainer_cls(config)


# Names the reference exports from its package root (landmark/__init__.py:4-19).  They are resolved on first access so
# that importing the package stays light for the configuration and data layers.
_LAZY = {
    "InferenceEngine": (".render.inference_engine", "InferenceEngine"),
    "InferenceInterface": (".render.inference_module", "InferenceInterface"),
    "InferenceModule": (".render.inference_module", "InferenceModule"),
    "InferenceModuleInitializer": (".render.initializer", "InferenceModuleInitializer"),
    "Model": (".components.model.base_model", "Model"),
    "init_communication_context": (".comm", "init_communication_context"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        value = getattr(importlib.import_module(module, __name__), attr)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["init_inference", "init_training", "Config", "EnvSetting", *_LAZY]

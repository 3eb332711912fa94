"""Kernel-runtime optimisation passes applied to an inference model (reference:
landmark/render/parallel_module/optimization_manager.py:1-54).  ``kernel_fusion`` swaps components for
their fused counterparts and turns on bf16 shadow grids; half precision and static allocation are
identity passes as in the reference."""
from __future__ import annotations

from ..convertor import ComponentConvertorFactory
from .inference_module import InferenceModule


class OptimizationManager:
    def __init__(self, config, merged_state_dict=None):
        self.config, self.merged_state_dict = config, merged_state_dict

    def _build_kernel_fusion(self, model):
        inner = model.inter_model if isinstance(model, InferenceModule) else model
        inner = ComponentConvertorFactory.get_convertor("runtime").convert(inner, self.config)
        if isinstance(model, InferenceModule):
            model.inter_model = inner
            return model
        return inner

    @staticmethod
    def _build_half_precision(model):
        return model

    @staticmethod
    def _build_static_allocation(model):
        return model

    def build(self, model):
        if self.config.get("kernel_fusion", False):
            model = self._build_kernel_fusion(model)
        if self.config.get("half_precision", False):
            model = self._build_half_precision(model)
        if self.config.get("static_allocation", False):
            model = self._build_static_allocation(model)
        return model

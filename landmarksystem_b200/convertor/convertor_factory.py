"""Component convertors: re-instantiate mapped components as their parallel or fused subclass
(reference: landmark/nerf_components/components_convertor/{convertor_factory.py:15-127,
parallelize.py:9-78, fusion.py:7-89}).

Replicated (non-partitioned) children are *not* wrapped in per-module DDP as the reference does for
branch parallel (parallelize.py:65-69): their gradients are synchronised explicitly by
:class:`landmarksystem_b200.parallel.grad_sync.GradSynchronizer`, which survives parameter
replacement (grid upsampling) without re-wrapping.
"""
from __future__ import annotations

import torch
from torch import nn

from ..components.model.base_module import BaseModule


def _reinstantiate(module: BaseModule, new_cls, **extra):
    kwargs = module.get_init_kwargs()
    kwargs.update(extra)
    new = new_cls(**kwargs)
    return new


class BaseConvertor:
    def convert(self, model: nn.Module, config, state_dict=None, verbose: bool = False) -> nn.Module:
        """``state_dict``: a full checkpoint to load into the model before the conversion (the reference passes the
        state it wants the converted components to start from, convertor_factory.py:77-127); ``verbose`` prints the
        class swaps."""
        raise NotImplementedError

    @staticmethod
    def _preload(model, state_dict):
        if state_dict is not None:
            loader = getattr(model, "load_from_state_dict", None)
            loader(state_dict, False) if loader is not None else model.load_state_dict(state_dict, strict=False)


class ParallelConvertor(BaseConvertor):
    def convert(self, model, config, state_dict=None, verbose: bool = False):
        from .convert_maps import PARALLEL_MAPS

        self._preload(model, state_dict)

        if getattr(config, "channel_parallel", False):
            table, degree = PARALLEL_MAPS["ChannelParallel"], int(config.channel_parallel_size)
        elif getattr(config, "branch_parallel", False):
            table, degree = PARALLEL_MAPS["BranchParallel"], int(config.plane_division[0] * config.plane_division[1])
        else:
            return model
        part, group = int(config.mp_rank), config.mp_group
        for name, child in list(model.named_children()):
            new_cls = table.get(type(child))
            if new_cls is None:
                continue
            init_state = None
            if not isinstance(child, new_cls) and getattr(config, "channel_parallel", False):
                init_state = {k: v for k, v in child.state_dict().items()}   # slice the already-built full grids
            elif getattr(child, "_loaded_full_state", None) is not None:
                init_state = child._loaded_full_state
            new = _reinstantiate(child, new_cls, parallel_degree=degree, parallel_part=part, group=group,
                                 init_state_dict=init_state)
            if getattr(child, "use_shadow", False):
                new.enable_shadow(getattr(config, "fused_optimizer", True), getattr(child, "lazy", False))
            if verbose:
                print(f"{name}: {type(child).__name__} -> {new_cls.__name__} (part {part} of {degree})", flush=True)
            setattr(model, name, new)
        return model


class RuntimeConvertor(BaseConvertor):
    """``runtime == "Kernel"``: swap components for their fused counterparts, keeping the weights."""

    def convert(self, model, config=None, state_dict=None, verbose: bool = False):
        from .convert_maps import KERNEL_FUSION_MAP

        self._preload(model, state_dict)

        def walk(parent):
            for name, child in list(parent.named_children()):
                new_cls = KERNEL_FUSION_MAP.get(type(child))
                if new_cls is not None:
                    new = _reinstantiate(child, new_cls)
                    new.load_state_dict(child.state_dict(), strict=False)
                    new.to(next(child.parameters()).device if any(True for _ in child.parameters()) else "cpu")
                    if verbose:
                        print(f"{name}: {type(child).__name__} -> {new_cls.__name__}", flush=True)
                    setattr(parent, name, new)
                else:
                    walk(child)
                if hasattr(child, "use_fused"):
                    child.use_fused = True
            if hasattr(parent, "use_fused"):
                parent.use_fused = True

        walk(model)
        for mod in model.modules():
            if type(mod).__name__ == "RGBDecoder":
                mod.use_fused = True
        return model


class ComponentConvertorFactory:
    _TABLE = {"parallelize": ParallelConvertor, "runtime": RuntimeConvertor}

    @staticmethod
    def get_convertor(convertor_type: str = None, convert_type: str = None) -> BaseConvertor:
        convertor_type = convertor_type if convertor_type is not None else convert_type    # the reference's keyword
        assert convertor_type in ComponentConvertorFactory._TABLE, f"unknown convertor '{convertor_type}'"
        return ComponentConvertorFactory._TABLE[convertor_type]()


ComponentsConvertorBase = BaseConvertor         # base-class name of the reference (components_convertor/convertor_factory.py)

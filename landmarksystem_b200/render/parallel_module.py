"""Parallel wrappers of the inference model (reference:
landmark/render/parallel_module/parallel_module.py:20-157): tensor (channel) parallel conversion and the
data-parallel scatter / gather of the leading (ray) dimension with zero padding.  Unlike the reference, which hands every
rank one contiguous band of rows, the rows are dealt round-robin (``parallel_config["dp_interleave"]``, default on) so that
the ranks' loads match."""
from __future__ import annotations

from typing import Any, Mapping

import torch
from torch.nn import Module

from ..comm import CommContext, ParallelMode, all_gather
from ..utils import Config
from .inference_module import InferenceModule
from .optimization_manager import OptimizationManager


class StageArgs:
    """Positional / keyword arguments flowing between schedule stages."""

    def __init__(self, args=(), kwargs=None):
        self.Args, self.Kwargs = tuple(args), dict(kwargs or {})


class ParallelModule(Module):
    def __init__(self, model: Module, config: Config) -> None:
        super().__init__()
        self._inference_config = config
        self._parallel_config = config.get("parallel_config") if hasattr(config, "get") else None
        self._dp_gap_size = 0
        self._gs_model = False
        self.model = self._parallize(model)

    def reset_dp_gap_size(self):
        self._dp_gap_size = 0

    def load_from_state_dict(self, state_dict: Mapping[str, Any], strict: bool = False):
        return self.model.load_from_state_dict(state_dict, strict)

    def _parallize(self, model: Module):
        raise NotImplementedError

    def _tp_size(self) -> int:
        return int(self._parallel_config.get("tp_size", 1)) if self._parallel_config is not None else 1

    def auto_tp(self, model):
        """Replace grid encodings by their channel-parallel versions (slices of the loaded full grids)."""
        from ..convertor import ComponentConvertorFactory

        assert isinstance(model, InferenceModule), "tensor parallel needs an InferenceModule"
        ctx = CommContext()
        cfg = Config(channel_parallel=True, channel_parallel_size=self._tp_size(),
                     mp_rank=ctx.get_local_rank(ParallelMode.TENSOR_PARALLEL),
                     mp_group=ctx.get_group(ParallelMode.TENSOR_PARALLEL), fused_optimizer=False)
        model.inter_model = ComponentConvertorFactory.get_convertor("parallelize").convert(model.inter_model, cfg)
        return model

    def _block_parallel(self) -> bool:
        return self._parallel_config is not None and self._parallel_config.get("mode", "channel") == "block"

    def auto_block(self, model):
        """Model parallelism by spatial blocks (``parallel_config = {"tp_size": N, "mode": "block"}``): every rank of the
        tensor-parallel group keeps one band of the scene's blocks and renders the ray segments inside it; the per-rank
        records are merged by the cross-GPU ordered composite (``parallel/mp_render.py``)."""
        from ..parallel.mp_render import ModelParallelRenderer, slice_model_to_block_window

        assert isinstance(model, InferenceModule), "block parallel needs an InferenceModule"
        ctx = CommContext()
        inner = model.inter_model
        slice_model_to_block_window(inner, ctx.get_local_rank(ParallelMode.TENSOR_PARALLEL), self._tp_size())
        inner._mp_renderer = ModelParallelRenderer(inner, max_rays=1 << 18, group=ctx.get_group(ParallelMode.TENSOR_PARALLEL))
        return model

    def preprocess(self, *args, **kwargs):
        return self.model.preprocess(*args, **kwargs)

    def postprocess(self, *args, **kwargs):
        return self.model.postprocess(*args, **kwargs)

    # -- data parallel over the leading dimension of the first argument ---------------------------------
    def _dp_layout(self):
        ctx = CommContext()
        world = ctx.get_world_size(ParallelMode.GLOBAL)
        dp = world // self._tp_size()
        return ctx, world, dp, world // dp

    def dp_scatter(self, stage_input):
        first = stage_input.Args[0]
        ctx, _, dp, stride = self._dp_layout()
        if dp == 1 or self._gs_model:
            return stage_input.Args, stage_input.Kwargs
        assert isinstance(first, torch.Tensor), "data-parallel scatter needs a tensor as first argument"
        part = ctx.get_global_rank() // stride
        gap = first.shape[0] % dp
        if gap > 0:
            self._dp_gap_size = dp - gap
            pad = torch.zeros((self._dp_gap_size, *first.shape[1:]), device=first.device, dtype=first.dtype)
            first = torch.cat((first, pad), dim=0)
        size = first.shape[0] // dp
        args = list(stage_input.Args)
        if self._dp_interleaved():
            # rows dealt round-robin: every rank gets a regular subsample of the image instead of one horizontal band, so
            # the ranks' loads match (rays near the horizon cross far more of the scene than rays looking down)
            args[0] = first[part::dp].contiguous()
        else:
            args[0] = first[part * size:(part + 1) * size]
        return tuple(args), stage_input.Kwargs

    def _dp_interleaved(self) -> bool:
        cfg = self._parallel_config
        return True if cfg is None else bool(cfg.get("dp_interleave", True))

    def dp_gather(self, stage_input):
        ctx, _, dp, stride = self._dp_layout()
        if dp == 1 or self._gs_model:
            return stage_input.Args, stage_input.Kwargs
        outs = []
        for single in stage_input.Args:
            if not isinstance(single, torch.Tensor):
                outs.append(single)
                continue
            single = single.contiguous()
            gathered = torch.empty((single.shape[0] * dp, *single.shape[1:]), dtype=single.dtype, device=single.device)
            if ctx.get_global_rank() % stride == 0:
                all_gather(gathered, single, comm_mode=ParallelMode.DATA_PARALLEL)
            if self._dp_interleaved():             # rank-major blocks back to the original row order
                gathered = gathered.view(dp, single.shape[0], *single.shape[1:]).transpose(0, 1).reshape(gathered.shape)
            if self._dp_gap_size > 0:
                gathered = gathered[: -self._dp_gap_size]
            outs.append(gathered)
        self.reset_dp_gap_size()
        return tuple(outs), stage_input.Kwargs

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)


class TorchParallelModule(ParallelModule):
    def _parallize(self, model: Module):
        if self._tp_size() > 1:
            return self.auto_block(model) if self._block_parallel() else self.auto_tp(model)
        return model


class KernelParallelModule(ParallelModule):
    def __init__(self, model: Module, config: Config, merged_state_dict=None) -> None:
        self.merged_state_dict = merged_state_dict
        super().__init__(model, config)

    def _parallize(self, model: Module):
        if self._tp_size() > 1:
            model = self.auto_block(model) if self._block_parallel() else self.auto_tp(model)
        return OptimizationManager(self._inference_config, self.merged_state_dict).build(model)

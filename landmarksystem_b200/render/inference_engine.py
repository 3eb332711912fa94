"""Inference engine: loads the checkpoint, wraps the model (dynamic loading, tensor / data parallel,
kernel runtime) and executes the static instruction list on every call (reference:
landmark/render/inference_engine/inference_engine.py:31-138).  Rank 0 calls ``engine(*args)``; other
ranks call ``engine()`` and receive the arguments through the gloo object broadcast."""
from __future__ import annotations

import torch
from torch.nn import Module

from ..comm import init_communication_context
from ..comm.collective import _broadcast_user_inputs_message
from ..utils import Config, _OFFLOAD_CONFIG_STR, _PARALLEL_CONFIG_STR
from .inference_module import InferenceInterface, InferenceModule
from .instructions import (BroadcastInputsInstruction, CallInstruction, DefModInstruction, DPGatherInstruction,
                           DPScatterInstruction, PipeGetResultInstruction, PipeSubmitInstruction, PostprocessInstruction,
                           PreprocessInstruction)
from .parallel_module import KernelParallelModule, StageArgs, TorchParallelModule
from .sches import gen_scheduler
from .types import RuntimeType


def _bind_default_stages(model: Module) -> None:
    if not hasattr(model, "preprocess"):
        model.preprocess = lambda *a, **k: (a, k)
    if not hasattr(model, "postprocess"):
        model.postprocess = lambda *a, **k: a[0] if len(a) == 1 and not k else a


class InferenceEngine(Module):
    def __init__(self, model: Module, config: Config) -> None:
        super().__init__()
        self.model = model
        if isinstance(model, InferenceModule):
            self.base_model = model.inter_model
        else:
            _bind_default_stages(model)
            self.base_model = model
        self._config = config
        self._parallel = config.get(_PARALLEL_CONFIG_STR) is not None
        self._model_initialized = False
        self._stage_input = StageArgs()
        self._inference_output = None
        self._pipe = None
        if self._parallel:
            init_communication_context(config.parallel_config)
        self.sche_list = gen_scheduler(config).steps()
        self.device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._exec_init()

    # -- instruction handlers -------------------------------------------------------------------------------
    def _exec_init(self):
        if self._model_initialized:
            return
        cfg = self._config
        self.model.eval()
        merged = None
        if cfg.get("ckpt_path") is not None:
            merged = self.model.get_state_dict_from_ckpt(cfg.ckpt_path, "cpu")
        if cfg.get(_OFFLOAD_CONFIG_STR) is not None:
            from .offload.offload_module import OffloadModule

            assert merged is not None, "dynamic loading needs a checkpoint"
            self.model = OffloadModule(self.model, merged_state_dict=merged, config=cfg.offload_config, device=self.device)
        elif merged is not None:
            self.model.load_from_state_dict(merged)
        runtime = RuntimeType(cfg.get("runtime", "Torch"))
        if runtime is RuntimeType.Kernel:
            self.model = KernelParallelModule(self.model, cfg, merged)
        else:
            self.model = TorchParallelModule(self.model, cfg)
        self.model.to(self.device)
        self._move_aux(self.device)
        self.model.eval()
        self._model_initialized = True

    def _move_aux(self, device):
        """Plain tensor attributes (AABBs, scene manager, alpha mask) that ``.to()`` does not reach."""
        for mod in self.model.modules():
            for name, value in list(vars(mod).items()):
                if name.startswith("_"):
                    continue
                if torch.is_tensor(value) and not isinstance(value, torch.nn.Parameter) and value.device != device:
                    setattr(mod, name, value.to(device))
                elif hasattr(value, "update_device"):
                    value.update_device(device)
                elif type(value).__name__ == "SceneManager":
                    value.to(device)
            if "device" in vars(mod):
                mod.device = device
        if device.type == "cuda" and RuntimeType(self._config.get("runtime", "Torch")) is RuntimeType.Kernel \
                and self._config.get(_OFFLOAD_CONFIG_STR) is None:
            # kernel runtime reads bf16 shadows of the feature grids (with dynamic loading the streamed window is the
            # storage the kernels read, in the dtype the offload configuration asks for: no second copy)
            for mod in self.model.modules():
                if hasattr(mod, "enable_shadow") and hasattr(mod, "plane_coef"):
                    mod.enable_shadow(False)

    @torch.no_grad()
    def _exec_forward(self):
        out = self.model.forward(*self._stage_input.Args, **self._stage_input.Kwargs)
        self._stage_input = StageArgs(out if isinstance(out, tuple) else (out,), {})

    def _exec_broadcast_inputs(self):
        payload = _broadcast_user_inputs_message([self._stage_input.Args, self._stage_input.Kwargs])
        self._stage_input = StageArgs(payload[0], payload[1])

    def _exec_dp_scatter(self):
        self._stage_input = StageArgs(*self.model.dp_scatter(self._stage_input))

    def _exec_dp_gather(self):
        self._stage_input = StageArgs(*self.model.dp_gather(self._stage_input))

    def _exec_preprocess(self):
        out = self.model.preprocess(*self._stage_input.Args, **self._stage_input.Kwargs)
        self._stage_input = StageArgs(out[0], out[1])

    def _exec_postprocess(self):
        self._inference_output = self.model.postprocess(*self._stage_input.Args, **self._stage_input.Kwargs)

    def _exec_pipe_submit(self):
        """Run the forward on the stage pipeline's worker (own CUDA stream) instead of the caller's."""
        from .easy_pipeline import EasyPipeRunner, PipelineItem

        if self._pipe is None:
            def call(item):
                with torch.no_grad():
                    out = self.model.forward(*item[0], **item[1])
                return out if isinstance(out, tuple) else (out,)

            self._pipe = EasyPipeRunner([PipelineItem(call, n_workers=1, use_cuda_stream=torch.cuda.is_available())])
        self._pipe.run_batch([(self._stage_input.Args, self._stage_input.Kwargs)])

    def _exec_pipe_get_result(self):
        self._stage_input = StageArgs(self._pipe.get_result(), {})

    _INSTRUCTION_MAP = {
        DefModInstruction: _exec_init, BroadcastInputsInstruction: _exec_broadcast_inputs,
        PreprocessInstruction: _exec_preprocess, DPScatterInstruction: _exec_dp_scatter,
        CallInstruction: _exec_forward, DPGatherInstruction: _exec_dp_gather,
        PostprocessInstruction: _exec_postprocess, PipeSubmitInstruction: _exec_pipe_submit,
        PipeGetResultInstruction: _exec_pipe_get_result,
    }

    def forward(self, *args, **kwargs):
        self._stage_input = StageArgs(args, kwargs)
        self._inference_output = None
        for step in self.sche_list:
            handler = self._INSTRUCTION_MAP.get(step)
            if handler is None:
                raise NotImplementedError(f"{step.__name__} not supported.")
            handler(self)
        return self._inference_output

    def close(self):
        if self._pipe is not None:
            self._pipe.stop()
            self._pipe = None

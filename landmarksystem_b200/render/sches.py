"""Static schedules: which instructions one engine call executes (reference:
landmark/render/scheduler/sches.py:20-135).  Single device: DefMod, Preprocess, Call, Postprocess;
multi device adds BroadcastInputs; data parallel adds DPScatter / DPGather around Call; the
pipelined variant submits the frame to the stage pipeline and collects the finished one."""
from __future__ import annotations

from typing import List

from ..utils import Config, EnvSetting, _OFFLOAD_CONFIG_STR, _PARALLEL_CONFIG_STR
from .instructions import (BroadcastInputsInstruction, CallInstruction, DefModInstruction, DPGatherInstruction,
                           DPScatterInstruction, Instruction, PipeGetResultInstruction, PipeSubmitInstruction,
                           PostprocessInstruction, PreprocessInstruction)


class AbstractSche:
    def steps(self, rank=None) -> List[type]:
        raise NotImplementedError


class InferenceSche(AbstractSche):
    def steps(self, rank=None):       # ``rank``: accepted as in the reference; the list is the same on every rank
        return [DefModInstruction, PreprocessInstruction, CallInstruction, PostprocessInstruction]


class MultiDeviceSche(InferenceSche):
    def steps(self, rank=None):       # ``rank``: accepted as in the reference; the list is the same on every rank
        return [DefModInstruction, BroadcastInputsInstruction, PreprocessInstruction, CallInstruction,
                PostprocessInstruction]


class DDPSche(MultiDeviceSche):
    def steps(self, rank=None):       # ``rank``: accepted as in the reference; the list is the same on every rank
        return [DefModInstruction, BroadcastInputsInstruction, PreprocessInstruction, DPScatterInstruction,
                CallInstruction, DPGatherInstruction, PostprocessInstruction]


class DDPPipeSche(DDPSche):
    def steps(self, rank=None):       # ``rank``: accepted as in the reference; the list is the same on every rank
        return [DefModInstruction, BroadcastInputsInstruction, PreprocessInstruction, DPScatterInstruction,
                PipeSubmitInstruction, PipeGetResultInstruction, DPGatherInstruction, PostprocessInstruction]


class DDPPipeOffloadSche(DDPPipeSche):
    pass


def gen_scheduler(config: Config) -> AbstractSche:
    world = EnvSetting.WORLD_SIZE
    par = config.get(_PARALLEL_CONFIG_STR) if hasattr(config, "get") else None
    if par is None or world == 1:
        return InferenceSche()
    tp = int(par.get("tp_size", 1))
    pipelined = bool(par.get("pipeline", False))
    if world // tp > 1:
        if pipelined:
            return DDPPipeOffloadSche() if config.get(_OFFLOAD_CONFIG_STR) is not None else DDPPipeSche()
        return DDPSche()
    return MultiDeviceSche()

"""Instruction markers of the static per-call render schedule (reference:
landmark/render/scheduler/instructions.py:1-53)."""


class Instruction:
    def __repr__(self) -> str:
        return type(self).__name__


class DefModInstruction(Instruction):
    """Build / load the model (no-op after the first call)."""


class CheckSyncInstruction(Instruction):
    """Agree across ranks on a dynamic-loading buffer swap."""


class CallInstruction(Instruction):
    """Run the model forward."""


class PipeSubmitInstruction(Instruction):
    """Hand the frame to the stage pipeline."""


class PipeGetResultInstruction(Instruction):
    """Fetch a finished frame from the stage pipeline."""


class BroadcastInputsInstruction(Instruction):
    """Send rank 0's call arguments to every rank."""


class PreprocessInstruction(Instruction):
    pass


class PostprocessInstruction(Instruction):
    pass


class DPGatherInstruction(Instruction):
    pass


class DPScatterInstruction(Instruction):
    pass

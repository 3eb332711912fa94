"""Names of the process groups the framework registers."""
from enum import Enum


class ParallelMode(str, Enum):
    GLOBAL = "global"
    DATA_PARALLEL = "data_parallel"
    TENSOR_PARALLEL = "tensor_parallel"
    MESSAGE_TRANSFER = "message_transfer"   # gloo group for pickled python objects
    DYNAMIC_LOAD = "dynamic_load"           # ranks that receive the same streamed scene blocks


CommMode = ParallelMode

"""Distributed communication layer: group registry, collective wrappers, differentiable collectives."""
from .collective import all_gather, all_reduce, broadcast, broadcast_object_list, gather, scatter
from .comm_context import CommContext, destroy_communication_context, init_communication_context
from .modes import CommMode, ParallelMode
from .train_groups import init_train_groups

__all__ = ["all_gather", "all_reduce", "broadcast", "broadcast_object_list", "gather", "scatter", "CommContext",
           "destroy_communication_context", "init_communication_context", "CommMode", "ParallelMode",
           "init_train_groups"]

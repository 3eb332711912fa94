"""Rank algebra of the render-side process groups (reference:
landmark/communicator/group_initializer.py:50-148).

Every initializer has a pure ``layout()`` that returns *all* groups as rank lists (testable without
``torch.distributed``) and ``init_dist_group()`` that creates them collectively and returns
``(local_rank, group_size, process_group, ranks, mode)`` for the calling rank.
"""
from __future__ import annotations

from typing import List, Optional

import torch.distributed as dist

from .modes import ParallelMode


class GroupInitializer:
    mode: ParallelMode
    backend: Optional[str] = None

    def __init__(self, rank: int, world_size: int):
        self.rank, self.world_size = rank, world_size

    def layout(self) -> List[List[int]]:
        raise NotImplementedError

    def init_dist_group(self):
        mine = None
        for ranks in self.layout():
            group = dist.new_group(ranks, backend=self.backend) if self.backend else dist.new_group(ranks)
            if self.rank in ranks:
                mine = (ranks.index(self.rank), len(ranks), group, ranks, self.mode)
        if mine is None:  # this rank takes no part in the mode (e.g. non-leading TP ranks for DP)
            mine = (None, 0, None, [], self.mode)
        return mine


class DPGroupInitializer(GroupInitializer):
    """One group holding the first rank of every tensor-parallel group."""
    mode = ParallelMode.DATA_PARALLEL

    def __init__(self, rank, world_size, data_parallel_size):
        super().__init__(rank, world_size)
        self.dp = data_parallel_size
        self.tp = world_size // data_parallel_size

    def layout(self):
        return [[i * self.tp for i in range(self.dp)]]


class TPGroupInitializer(GroupInitializer):
    """Contiguous blocks of ``tensor_parallel_size`` ranks."""
    mode = ParallelMode.TENSOR_PARALLEL

    def __init__(self, rank, world_size, tensor_parallel_size):
        super().__init__(rank, world_size)
        self.tp = tensor_parallel_size

    def layout(self):
        return [list(range(s, s + self.tp)) for s in range(0, self.world_size, self.tp)]


class MessageTransferInitializer(GroupInitializer):
    """All ranks on the gloo backend: carries pickled user inputs."""
    mode = ParallelMode.MESSAGE_TRANSFER
    backend = "gloo"

    def layout(self):
        return [list(range(self.world_size))]


class DynamicLoadGroupInitializer(GroupInitializer):
    """For each tensor-parallel offset, the ranks with that offset, split per node: the first rank of
    each group copies a block host-to-device and fans it out to the others."""
    mode = ParallelMode.DYNAMIC_LOAD

    def __init__(self, rank, world_size, tensor_parallel_size, node_cuda_num):
        super().__init__(rank, world_size)
        self.tp = tensor_parallel_size
        self.per_node = max(int(node_cuda_num), 1)

    def layout(self):
        groups = []
        n_nodes = (self.world_size + self.per_node - 1) // self.per_node
        for offset in range(self.tp):
            same = list(range(offset, self.world_size, self.tp))
            for node in range(n_nodes):
                lo, hi = node * self.per_node, (node + 1) * self.per_node
                ranks = [r for r in same if lo <= r < hi]
                if ranks:
                    groups.append(ranks)
        return groups


ProcessGroupInitializer = GroupInitializer      # base-class name of the reference (communicator/group_initializer.py)

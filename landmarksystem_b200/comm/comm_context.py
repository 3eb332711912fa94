"""Singleton registry of process groups (reference: landmark/communicator/comm_context.py:18-162).

Bootstrap, object broadcast and barriers stay on ``torch.distributed`` (NCCL for tensors, gloo for
pickled objects).  The hot-path collectives of the fused kernels use peer memory instead
(:mod:`landmarksystem_b200.comm.symmetric`).
"""
from __future__ import annotations

import datetime
import gc
import os

import torch
import torch.distributed as dist

from ..utils import Config, EnvSetting, SingletonMeta, _RANK_STR, _WORLD_SIZE_STR
from .group_initializer import (DPGroupInitializer, DynamicLoadGroupInitializer, MessageTransferInitializer,
                                TPGroupInitializer)
from .modes import CommMode


def default_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


class CommContext(metaclass=SingletonMeta):
    def __init__(self) -> None:
        self._local_ranks, self._global_ranks, self._world_sizes = {}, {}, {}
        self._ranks_in_group, self._groups = {}, {}
        self._node_cuda_num = max(torch.cuda.device_count(), 1)
        self._tensor_parallel_size = 1
        self._data_parallel_size = 1
        self._owns_pg = False

    def is_initialized(self) -> bool:
        return self._groups.get(CommMode.GLOBAL) is not None

    def init_distributed_env(self, world_size=None, rank=None, backend=None, dist_url="env://", timeout=1800):
        backend = backend or default_backend()
        if not dist.is_initialized():
            dist.init_process_group(backend=backend, init_method=dist_url, world_size=world_size, rank=rank,
                                    timeout=datetime.timedelta(seconds=timeout))
            self._owns_pg = True
        world_size, rank = dist.get_world_size(), dist.get_rank()
        if torch.cuda.is_available():
            local = int(os.environ.get("LOCAL_RANK", rank % torch.cuda.device_count()))
            torch.cuda.set_device(local % torch.cuda.device_count())
        dist.barrier()
        self._register_group(rank, world_size, dist.group.WORLD, list(range(world_size)), CommMode.GLOBAL)
        self._global_ranks[CommMode.GLOBAL] = rank

    def _register_group(self, local_rank, world_size, process_group, ranks_in_group, mode):
        self._local_ranks[mode] = local_rank
        self._world_sizes[mode] = world_size
        self._groups[mode] = process_group
        self._ranks_in_group[mode] = ranks_in_group

    def get_group(self, comm_mode: CommMode):
        return self._groups[comm_mode]

    def get_world_size(self, comm_mode: CommMode):
        return self._world_sizes[comm_mode]

    def get_global_rank(self):
        return self._global_ranks[CommMode.GLOBAL]

    def get_local_rank(self, comm_mode: CommMode):
        return self._local_ranks[comm_mode]

    def get_ranks_in_group(self, comm_mode: CommMode):
        return self._ranks_in_group[comm_mode]

    @property
    def tensor_parallel_size(self):
        return self._tensor_parallel_size

    @property
    def data_parallel_size(self):
        return self._data_parallel_size

    def init_groups(self, config: Config):
        rank = self.get_global_rank()
        world = self.get_world_size(CommMode.GLOBAL)
        self._tensor_parallel_size = int(config.get("tp_size", 1)) if hasattr(config, "get") else 1
        assert world % self._tensor_parallel_size == 0, "world size must be a multiple of tp_size"
        self._data_parallel_size = world // self._tensor_parallel_size
        for init in (DPGroupInitializer(rank, world, self._data_parallel_size),
                     TPGroupInitializer(rank, world, self._tensor_parallel_size),
                     MessageTransferInitializer(rank, world),
                     DynamicLoadGroupInitializer(rank, world, self._tensor_parallel_size, self._node_cuda_num)):
            self._register_group(*init.init_dist_group())

    def destroy(self):
        if not self.is_initialized():
            return
        dist.barrier()
        if self._owns_pg:
            dist.destroy_process_group()
        for d in (self._local_ranks, self._global_ranks, self._world_sizes, self._ranks_in_group, self._groups):
            d.clear()
        self._tensor_parallel_size = self._data_parallel_size = 1
        self._owns_pg = False
        gc.collect()


def init_communication_context(parallel_config: Config, backend: str = None, dist_url: str = "env://"):
    ctx = CommContext()
    if ctx.is_initialized():
        return
    assert hasattr(parallel_config, _RANK_STR) and hasattr(parallel_config, _WORLD_SIZE_STR)
    ctx.init_distributed_env(world_size=parallel_config.world_size, rank=parallel_config.rank, backend=backend,
                             dist_url=dist_url, timeout=EnvSetting.COMM_TIMEOUT)
    ctx.init_groups(parallel_config)


def destroy_communication_context():
    CommContext().destroy()

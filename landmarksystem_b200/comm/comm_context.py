"""Singleton registry of process groups (reference: landmark/communicator/comm_context.py:18-162).

Bootstrap, object broadcast and barriers stay on ``torch.distributed`` (NCCL for tensors, gloo for
pickled objects).  The hot-path collectives of the fused kernels use peer memory instead
(:mod:`landmarksystem_b200.comm.symmetric`).
"""
from __future__ import annotations

import dataclasses
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


@dataclasses.dataclass(frozen=True)
class GroupRecord:
    """What the context knows about one communication mode on this process."""

    rank_in_group: int
    size: int
    group: object              # torch.distributed process group handle
    members: tuple             # global ranks of the group, in group order


class CommContext(metaclass=SingletonMeta):
    """One ``{mode: GroupRecord}`` map behind the reference's accessor names."""

    def __init__(self) -> None:
        self._records: dict = {}
        self._rank = None
        self._node_cuda_num = max(torch.cuda.device_count(), 1)
        self._tp = self._dp = 1
        self._owns_pg = False

    def is_initialized(self) -> bool:
        return CommMode.GLOBAL in self._records

    def init_distributed_env(self, world_size=None, rank=None, backend=None, dist_url="env://", timeout=1800):
        if not dist.is_initialized():
            dist.init_process_group(backend=backend or default_backend(), init_method=dist_url, world_size=world_size,
                                    rank=rank, timeout=datetime.timedelta(seconds=timeout))
            self._owns_pg = True
        self._rank = dist.get_rank()
        n = dist.get_world_size()
        if torch.cuda.is_available():
            ndev = torch.cuda.device_count()
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", self._rank % ndev)) % ndev)
        dist.barrier()
        self._records[CommMode.GLOBAL] = GroupRecord(self._rank, n, dist.group.WORLD, tuple(range(n)))

    def _record(self, comm_mode: CommMode) -> GroupRecord:
        try:
            return self._records[comm_mode]
        except KeyError:
            raise KeyError(f"communication mode {comm_mode} has no group on this process") from None

    # accessor names are the reference's public surface
    def get_group(self, comm_mode: CommMode):
        return self._record(comm_mode).group

    def get_world_size(self, comm_mode: CommMode):
        return self._record(comm_mode).size

    def get_global_rank(self):
        return self._rank

    def get_local_rank(self, comm_mode: CommMode):
        return self._record(comm_mode).rank_in_group

    def get_ranks_in_group(self, comm_mode: CommMode):
        return list(self._record(comm_mode).members)

    @property
    def tensor_parallel_size(self):
        return self._tp

    @property
    def data_parallel_size(self):
        return self._dp

    def init_groups(self, config: Config):
        me, n = self._rank, self._record(CommMode.GLOBAL).size
        self._tp = int(config.get("tp_size", 1)) if hasattr(config, "get") else 1
        assert n % self._tp == 0, "world size must be a multiple of tp_size"
        self._dp = n // self._tp
        builders = (DPGroupInitializer(me, n, self._dp), TPGroupInitializer(me, n, self._tp),
                    MessageTransferInitializer(me, n), DynamicLoadGroupInitializer(me, n, self._tp, self._node_cuda_num))
        for builder in builders:
            rank_in_group, size, group, members, mode = builder.init_dist_group()
            self._records[mode] = GroupRecord(rank_in_group, size, group, tuple(members or ()))

    def destroy(self):
        if not self.is_initialized():
            return
        dist.barrier()
        if self._owns_pg:
            dist.destroy_process_group()
        self._records.clear()
        self._rank, self._tp, self._dp, self._owns_pg = None, 1, 1, False
        gc.collect()


def init_communication_context(parallel_config: Config, backend: str = None, dist_url: str = "env://"):
    ctx = CommContext()
    if ctx.is_initialized():
        # a trainer (or an earlier engine) of this process brought the context up: keep the process group, and build
        # the render-side groups if they are missing or were laid out for another tensor-parallel size
        want_tp = int(parallel_config.get("tp_size", 1)) if hasattr(parallel_config, "get") else 1
        if CommMode.DATA_PARALLEL not in ctx._records or ctx.tensor_parallel_size != want_tp:
            ctx.init_groups(parallel_config)
        return
    assert hasattr(parallel_config, _RANK_STR) and hasattr(parallel_config, _WORLD_SIZE_STR)
    ctx.init_distributed_env(world_size=parallel_config.world_size, rank=parallel_config.rank, backend=backend,
                             dist_url=dist_url, timeout=EnvSetting.COMM_TIMEOUT)
    ctx.init_groups(parallel_config)


def destroy_communication_context():
    CommContext().destroy()

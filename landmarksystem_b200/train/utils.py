"""Small trainer helpers (reference: landmark/train/utils/utils.py:1-43 and
landmark/train/utils/distributed_utils.py:14-227)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


class CircularIterator:
    """Cycle over a list forever."""

    def __init__(self, items):
        self.items, self.pos = list(items), 0

    def __iter__(self):
        return self

    def __next__(self):
        item = self.items[self.pos]
        self.pos = (self.pos + 1) % len(self.items)
        return item


def rm_redundant_words_in_state_dict(state_dict, words):
    """Drop every occurrence of the given substrings (e.g. ``"module."``) from state-dict keys."""
    out = {}
    for key, value in state_dict.items():
        for word in words:
            key = key.replace(word, "")
        out[key] = value
    return out


class st:
    """ANSI colours for console messages."""
    RESET, BOLD, RED, GREEN, YELLOW, BLUE = "\033[0m", "\033[1m", "\033[31m", "\033[32m", "\033[33m", "\033[34m"


def get_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else int(os.environ.get("RANK", 0))


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", os.environ.get("SLURM_LOCALID", 0)))


def is_main_rank() -> bool:
    return get_rank() == 0


def init_distributed_mode(env: str = "single_node", backend: str = None, timeout_s: int = 1800) -> dict:
    """Bring up ``torch.distributed`` from the launcher's environment and return ``{rank, world_size, local_rank}``
    (reference: landmark/train/utils/distributed_utils.py:73-140).  ``env``: ``"single_node"`` / ``"torchrun"`` read
    ``RANK / WORLD_SIZE / LOCAL_RANK``; ``"slurm"`` derives them from ``SLURM_PROCID / SLURM_NTASKS / SLURM_LOCALID`` and
    takes the first host of ``SLURM_NODELIST`` as master; ``"aliyun"`` reads the DLC launcher's ``RANK`` (node rank),
    ``WORLD_SIZE`` (node count) and ``LOCAL_RANK`` with ``NPROC_PER_NODE`` processes per node.  Idempotent.

    The reference passes its configuration object: ``init_distributed_mode(args)`` reads ``args.env`` and writes
    ``args.rank / args.world_size / args.local_rank / args.distributed`` back."""
    import datetime

    if not isinstance(env, str):
        args = env
        info = init_distributed_mode(str(getattr(args, "env", None) or "single_node"), backend, timeout_s)
        for key, value in info.items():
            setattr(args, key, value)
        args.distributed = info["world_size"] > 1
        return info

    if env == "slurm":
        rank, world = int(os.environ["SLURM_PROCID"]), int(os.environ["SLURM_NTASKS"])
        local = int(os.environ.get("SLURM_LOCALID", 0))
        nodelist = os.environ.get("SLURM_NODELIST", "127.0.0.1")
        first = nodelist.split(",")[0]
        if "[" in first:                                  # "node[03-07]" -> "node03"
            head, rng = first.split("[", 1)
            first = head + rng.rstrip("]").split("-")[0].split(",")[0]
        os.environ.setdefault("MASTER_ADDR", first)
        os.environ.setdefault("MASTER_PORT", "29501")
    elif env == "aliyun":
        per_node = int(os.environ.get("NPROC_PER_NODE", max(torch.cuda.device_count(), 1)))
        local = int(os.environ.get("LOCAL_RANK", 0))
        rank = int(os.environ.get("RANK", 0)) * per_node + local
        world = int(os.environ.get("WORLD_SIZE", 1)) * per_node
    else:
        rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
        local = int(os.environ.get("LOCAL_RANK", 0))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(local))
    if world > 1 and not dist.is_initialized():
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        if torch.cuda.is_available():
            torch.cuda.set_device(local % torch.cuda.device_count())
        dist.init_process_group(backend=backend, init_method="env://", world_size=world, rank=rank,
                                timeout=datetime.timedelta(seconds=timeout_s))
        dist.barrier()
    return {"rank": rank, "world_size": world, "local_rank": local}


# -- process-wide group registry under the reference's function names (landmark/train/utils/distributed_utils.py:
# 14-70, 171-227).  The trainers keep their groups on the run configuration (``comm/train_groups.py``); these helpers
# serve scripts written against the module-level interface. ------------------------------------------------------
_GROUPS = {"dp": None, "mp": None, "mp_ranks": [0], "mp_part": 0}


def is_dist_avail_and_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def is_main_process() -> bool:
    return get_rank() == 0


def get_local_size() -> int:
    """Ranks on this node (``LOCAL_SIZE`` / ``LOCAL_WORLD_SIZE`` of the launcher); 1 outside a distributed run."""
    if not is_dist_avail_and_initialized():
        return 1
    return int(os.environ.get("LOCAL_SIZE", os.environ.get("LOCAL_WORLD_SIZE", 1)))


def save_on_master(*args, **kwargs) -> None:
    if is_main_rank():
        torch.save(*args, **kwargs)


def setup_for_distributed(is_master: bool):
    """Silence ``print`` on every rank but the master's (``print(..., force=True)`` still prints everywhere).
    Returns the original ``print`` so that a caller can restore it."""
    import builtins

    original = builtins.print

    def rank_print(*args, **kwargs):
        if kwargs.pop("force", False) or is_master:
            original(*args, **kwargs)

    builtins.print = rank_print
    return original


def init_comm_groups(model_parallel_degree: int = 8) -> None:
    """Contiguous model-parallel groups of ``model_parallel_degree`` ranks and the data-parallel groups strided
    across them; every rank creates every group (collective) and keeps its own two."""
    from ..comm.train_groups import group_layout

    assert dist.is_initialized(), "initialise torch.distributed first"
    rank = dist.get_rank()
    mp_groups, dp_groups = group_layout(dist.get_world_size(), model_parallel_degree)
    for ranks in mp_groups:
        group = dist.new_group(ranks)
        if rank in ranks:
            _GROUPS["mp"], _GROUPS["mp_ranks"] = group, list(ranks)
    for ranks in dp_groups:
        group = dist.new_group(ranks)
        if rank in ranks:
            _GROUPS["dp"] = group
    _GROUPS["mp_part"] = rank % model_parallel_degree


def get_dp_group():
    return _GROUPS["dp"]


def get_mp_group():
    return _GROUPS["mp"]


def get_mp_rank0() -> int:
    return _GROUPS["mp_ranks"][0]


def get_mp_part() -> int:
    return _GROUPS["mp_part"]

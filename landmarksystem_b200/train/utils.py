"""Small trainer helpers (reference: landmark/train/utils/utils.py:1-43 and
landmark/train/utils/distributed_utils.py:14-227)."""
from __future__ import annotations

import os

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

"""Pre-processed ray shards: ``num.npz`` + ``%010d.npz{rays[8192,6], rgbs[8192,3], idxs[8192]}``
(reference: .../dataloader/processeddataset.py:6-72)."""
from __future__ import annotations

import os

import numpy as np
import torch
from torch.utils.data import Dataset


class PreprocessedDataset(Dataset):
    shard_rays = 8192

    def __init__(self, root: str, data_type: str = "file"):
        assert data_type == "file", "only file-backed shards are supported (no object store offline)"
        self.root = root
        self.num = int(np.load(os.path.join(root, "num.npz"))["num"])

    def __len__(self):
        return self.num

    def __getitem__(self, i):
        shard = np.load(os.path.join(self.root, f"{i:010d}.npz"))
        return (torch.from_numpy(shard["rays"]).float(), torch.from_numpy(shard["rgbs"]).float(),
                torch.from_numpy(shard["idxs"]).float())


def write_shards(root: str, rays: torch.Tensor, rgbs: torch.Tensor, idxs: torch.Tensor, shard_rays: int = 8192):
    """Shuffle and write full shards; returns ``(n_shards, leftover_tuple)`` (leftovers are gathered
    across ranks by the distributed preprocessors, reference: city_dataset.py:437-439)."""
    os.makedirs(root, exist_ok=True)
    perm = torch.randperm(rays.shape[0])
    rays, rgbs, idxs = rays[perm], rgbs[perm], idxs[perm]
    n = rays.shape[0] // shard_rays
    for k in range(n):
        s = slice(k * shard_rays, (k + 1) * shard_rays)
        np.savez(os.path.join(root, f"{k:010d}.npz"), rays=rays[s].numpy(), rgbs=rgbs[s].numpy(), idxs=idxs[s].numpy())
    np.savez(os.path.join(root, "num.npz"), num=n)
    tail = slice(n * shard_rays, None)
    return n, (rays[tail], rgbs[tail], idxs[tail])

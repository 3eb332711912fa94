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
        if self.num > 0:                          # shards written with another size than the default
            with np.load(os.path.join(root, f"{0:010d}.npz")) as first:
                self.shard_rays = int(first["idxs"].shape[0])

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


def preprocess(dataset, root: str, shard_rays: int = 8192) -> int:
    """Single-process shard writer for a ``VolumeRenderDataset`` (all rays in memory): shuffles, writes the full
    shards and drops the incomplete tail.  Returns the number of shards."""
    n, _ = write_shards(root, dataset.all_rays, dataset.all_rgbs, dataset.all_idxs, shard_rays)
    return n


def dist_preprocess(dataset, root: str, rank: int, world: int, shard_rays: int = 8192, group=None) -> int:
    """Distributed shard writer (reference: city_dataset.py:380-460): the rays are split evenly between the ranks,
    each rank shuffles and writes its full shards under globally unique numbers, the incomplete tails are gathered on
    rank 0 (``all_gather_object`` - host objects, gloo or nccl) and written as extra shards there; ``num.npz`` holds
    the total.  Returns the total number of shards (same on every rank)."""
    import torch.distributed as dist

    os.makedirs(root, exist_ok=True)
    total = dataset.all_rays.shape[0]
    lo, hi = total * rank // world, total * (rank + 1) // world
    g = torch.Generator().manual_seed(1234 + rank)
    perm = torch.randperm(hi - lo, generator=g) + lo
    rays, rgbs, idxs = dataset.all_rays[perm], dataset.all_rgbs[perm], dataset.all_idxs[perm]
    mine = (hi - lo) // shard_rays
    counts = [None] * world
    if world > 1:
        dist.all_gather_object(counts, mine, group=group)
    else:
        counts = [mine]
    first = sum(counts[:rank])
    for k in range(mine):
        s = slice(k * shard_rays, (k + 1) * shard_rays)
        np.savez(os.path.join(root, f"{first + k:010d}.npz"), rays=rays[s].numpy(), rgbs=rgbs[s].numpy(), idxs=idxs[s].numpy())
    tail = (rays[mine * shard_rays:].numpy(), rgbs[mine * shard_rays:].numpy(), idxs[mine * shard_rays:].numpy())
    tails = [None] * world
    if world > 1:
        dist.all_gather_object(tails, tail, group=group)
    else:
        tails = [tail]
    n_total = sum(counts)
    if rank == 0:
        r = np.concatenate([t[0] for t in tails]); c = np.concatenate([t[1] for t in tails]); i = np.concatenate([t[2] for t in tails])
        extra = r.shape[0] // shard_rays
        for k in range(extra):
            s = slice(k * shard_rays, (k + 1) * shard_rays)
            np.savez(os.path.join(root, f"{n_total + k:010d}.npz"), rays=r[s], rgbs=c[s], idxs=i[s])
        n_total += extra
        np.savez(os.path.join(root, "num.npz"), num=n_total)
    if world > 1:
        box = [n_total]
        dist.broadcast_object_list(box, src=0, group=group)
        n_total = box[0]
    return n_total

"""Dataset factories and the training ray sampler (reference:
landmark/nerf_components/data/datasets/dataloader/utils/dataset_utils.py:15-203)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class SimpleSampler:
    """Epoch-wise random permutation over ``total`` items served in batches; the generator is
    seeded so that every rank can draw the same sequence without a broadcast."""

    def __init__(self, total: int, batch: int, seed: Optional[int] = None):
        self.total, self.batch, self.curr = total, batch, total
        self.gen = torch.Generator()
        if seed is not None:
            self.gen.manual_seed(seed)
        self.ids = None

    def nextids(self) -> torch.Tensor:
        self.curr += self.batch
        if self.curr + self.batch > self.total:
            self.ids = torch.randperm(self.total, generator=self.gen)
            self.curr = 0
        return self.ids[self.curr:self.curr + self.batch]


class DistributedSampler:
    """Ray sampler of data-parallel training (reference: dataset_utils.py:41-62): every rank draws the same
    permutation of an epoch (seeded with ``seed + epoch``) and takes its own ``batch`` out of each stride of
    ``batch * world_size`` ids, so the ranks' batches of a step are disjoint."""

    def __init__(self, total: int, batch: int, rank: int, world_size: int, seed: int = 0):
        self.total, self.batch, self.rank, self.world_size, self.seed = total, batch, rank, world_size, seed
        self.curr, self.epoch, self.ids = total, 0, None

    def nextids(self) -> torch.Tensor:
        stride = self.batch * self.world_size
        self.curr += stride
        if self.ids is None or self.curr + stride > self.total:
            gen = torch.Generator()
            gen.manual_seed(self.seed + self.epoch)
            self.ids = torch.randperm(self.total, generator=gen)
            self.curr, self.epoch = 0, self.epoch + 1
        lo = self.curr + self.rank * self.batch
        return self.ids[lo:lo + self.batch]


class CameraDistributedSampler(torch.utils.data.distributed.DistributedSampler):
    """Per-rank camera order of data-parallel Gaussian training (``torch``'s sampler under a local name)."""


@dataclass
class DatasetInfo:
    aabb: torch.Tensor
    near_far: list
    white_bg: bool


def _dataset_cls(name: str, kind: str):
    from . import dataset_dict, gaussian_dataset_dict

    table = dataset_dict if kind == "nerf" else gaussian_dataset_dict
    assert name in table, f"unknown {kind} dataset '{name}' (known: {sorted(table)})"
    return table[name]


def prep_traindataset(enable_lpips, config):
    return _dataset_cls(config.dataset_name, "nerf")(split="train", downsample=config.downsample_train,
                                                     is_stack=enable_lpips, args=config, enable_lpips=enable_lpips)


def prep_testdataset(config):
    return _dataset_cls(config.dataset_name, "nerf")(split="test", downsample=config.downsample_train,
                                                     is_stack=True, args=config)


def prep_pathdataset(config):
    """The ``"path"`` split: a fly-around (``render_spherical``) or the frames of ``trajectories/path{id}.json``."""
    return _dataset_cls(config.dataset_name, "nerf")(split="path", downsample=config.downsample_train,
                                                     is_stack=True, args=config)


def prep_dataset(enable_lpips, config):
    return prep_traindataset(enable_lpips, config), prep_testdataset(config)


def prep_sampler(enable_lpips, config, train_dataset):
    allrays, allrgbs, allidxs = train_dataset.all_rays, train_dataset.all_rgbs, train_dataset.all_idxs
    if enable_lpips:  # patch sampling: one patch of patch_size^2 rays per step
        ps = config.patch_size
        W, H = train_dataset.img_wh
        n_img = allrays.shape[0]
        rays = allrays.view(n_img, H, W, 6).unfold(1, ps, ps).unfold(2, ps, ps)
        rays = rays.permute(0, 1, 2, 4, 5, 3).reshape(-1, ps * ps, 6)
        rgbs = allrgbs.view(n_img, H, W, 3).unfold(1, ps, ps).unfold(2, ps, ps)
        rgbs = rgbs.permute(0, 1, 2, 4, 5, 3).reshape(-1, ps * ps, 3)
        idxs = allidxs.view(n_img, H, W).unfold(1, ps, ps).unfold(2, ps, ps).reshape(-1, ps * ps)
        return rays, rgbs, idxs, SimpleSampler(rays.shape[0], 1, seed=config.random_seed)
    return allrays, allrgbs, allidxs, SimpleSampler(allrays.shape[0], config.batch_size, seed=config.random_seed)


def prep_traindataset_gs(config):
    return _dataset_cls(config.dataset_name, "gaussian")(split="train", downsample=config.downsample_train,
                                                         args=config, preload=config.preload)


def prep_testdataset_gs(config):
    return _dataset_cls(config.dataset_name, "gaussian")(split="test", downsample=config.downsample_train,
                                                         args=config, preload=config.preload)


def prep_dataset_gs(config):
    """``(train, test)`` camera datasets."""
    return prep_traindataset_gs(config), prep_testdataset_gs(config)


def PILtoTorch(pil_img) -> torch.Tensor:
    """A PIL image as a ``[C, H, W]`` tensor in [0, 1] (grey images get one channel)."""
    import numpy as np

    t = torch.from_numpy(np.array(pil_img)) / 255.0
    return t.permute(2, 0, 1) if t.dim() == 3 else t[None]


def getNeRFppNorm(cams) -> dict:
    """Centre and extent of a camera rig: ``translate`` = minus the mean camera centre, ``radius`` = 1.1 x the largest
    distance of a camera from that mean (the scene-extent convention of 3D Gaussian splatting)."""
    centres = torch.stack([torch.as_tensor(c.camera_center, dtype=torch.float32).cpu() for c in cams])
    mean = centres.mean(dim=0)
    radius = float((centres - mean).norm(dim=-1).max()) * 1.1
    return {"translate": (-mean).numpy(), "radius": radius}


def get_preprocessed_loader(config):
    """Loader over pre-computed ray shards.  Under data parallelism every replica (a model-parallel group when
    ``model_parallel_and_DDP``, else a rank) reads its own share of the shards and ``batch_size`` is divided among the
    replicas (reference: dataset_utils.py:147-176)."""
    from .processed_dataset import PreprocessedDataset

    ds = PreprocessedDataset(config.preprocessed_dir, config.processed_data_type)
    shards = max(config.batch_size // ds.shard_rays, 1)
    pin = torch.cuda.is_available()
    if config.get("DDP", False):
        if config.get("model_parallel_and_DDP", False):
            replicas, rank = int(config.get("num_mp_groups", 1) or 1), int(config.get("dp_rank", 0) or 0)
        else:
            replicas, rank = int(config.get("world_size", 1) or 1), int(config.get("rank", 0) or 0)
        if replicas > 1:
            sampler = CameraDistributedSampler(ds, num_replicas=replicas, rank=rank, shuffle=True, seed=0, drop_last=False)
            return torch.utils.data.DataLoader(ds, batch_size=max(shards // replicas, 1), sampler=sampler, num_workers=0,
                                               pin_memory=pin)
    return torch.utils.data.DataLoader(ds, batch_size=shards, shuffle=True, num_workers=0, pin_memory=pin)

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


class DistributedSampler(torch.utils.data.distributed.DistributedSampler):
    """Alias kept for API parity."""


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


def get_preprocessed_loader(config):
    from .processed_dataset import PreprocessedDataset

    ds = PreprocessedDataset(config.preprocessed_dir, config.processed_data_type)
    return torch.utils.data.DataLoader(ds, batch_size=max(config.batch_size // ds.shard_rays, 1), shuffle=True,
                                       num_workers=0, pin_memory=torch.cuda.is_available())

"""Dataset manager (reference: landmark/nerf_components/data/data_manager.py:20-329).

NeRF type: serves ray batches.  Unlike the reference - where rank 0 samples a batch and broadcasts
rays/rgb/idx to every rank each iteration (three NCCL broadcasts, data_manager.py:173-176) - every
rank builds the same seeded sampler and slices its own data-parallel share locally; the batch is
staged in pinned host memory and copied with one asynchronous H2D transfer.
Gaussian type: serves ``(Camera, image)`` pairs, optionally restricted to a spatial cell.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch.utils.data import ConcatDataset, DataLoader

from .datasets.dataset_utils import (CameraDistributedSampler, DatasetInfo, get_preprocessed_loader, prep_dataset,
                                     prep_sampler, prep_testdataset, prep_testdataset_gs, prep_traindataset,
                                     prep_traindataset_gs)


class DatasetManager:
    def __init__(self, config, enable_lpips: bool = False):
        self.config = config
        self.enable_lpips = enable_lpips
        self.iter_cnt = 0
        self._stage = None
        if config.dataset_type == "nerf":
            self._init_nerf()
        elif config.dataset_type == "gaussian":
            self._init_gaussian()
        else:
            raise ValueError(f"Unknown dataset type {config.dataset_type}")

    # -- NeRF ------------------------------------------------------------------------------
    def _init_nerf(self):
        cfg = self.config
        self.test_dataset = prep_testdataset(cfg)
        if cfg.is_train:
            if cfg.use_preprocessed_data:
                self.train_dataloader = get_preprocessed_loader(cfg)
                self._batch_iter = None
            else:
                self.train_dataset = prep_traindataset(self.enable_lpips, cfg)
                self.allrays, self.allrgbs, self.allidxs, self.trainingsampler = prep_sampler(
                    self.enable_lpips, cfg, self.train_dataset)
        self.dataset_info = DatasetInfo(self.test_dataset.scene_bbox, self.test_dataset.near_far,
                                        self.test_dataset.white_bg)
        self.white_bg = self.dataset_info.white_bg

    def _replica(self):
        cfg = self.config
        if not cfg.get("DDP", False):
            return 1, 0
        if cfg.get("model_parallel_and_DDP", False):
            return int(cfg.num_mp_groups), int(cfg.dp_rank)
        return int(cfg.get("world_size", 1)), int(cfg.get("rank", 0))

    _STAGES = 4

    def _to_device(self, rays, rgbs, idxs):
        """Pack into a pinned staging buffer -> one async H2D copy.  The staging buffers form a ring, each guarded
        by an event recorded after its copy: the host waits for that event before it overwrites the buffer, so a
        host thread that runs ahead of the GPU (a training step replayed from a CUDA graph costs it almost nothing)
        never rewrites a batch whose copy is still queued."""
        device = torch.device(self.config.device)
        packed = torch.cat((rays.reshape(-1, 6), rgbs.reshape(-1, 3), idxs.reshape(-1, 1)), dim=-1)
        if device.type != "cuda":
            return packed[:, :6], packed[:, 6:9], packed[:, 9]
        ring = self._stage
        if ring is None or ring["shape"] != packed.shape:
            ring = self._stage = {"shape": packed.shape, "next": 0, "events": [None] * self._STAGES,
                                  "bufs": [torch.empty(packed.shape, dtype=packed.dtype).pin_memory()
                                           for _ in range(self._STAGES)]}
        k = ring["next"]
        ring["next"] = (k + 1) % self._STAGES
        if ring["events"][k] is not None:
            ring["events"][k].synchronize()
        ring["bufs"][k].copy_(packed)
        dev = ring["bufs"][k].to(device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(device))
        ring["events"][k] = ev
        return dev[:, :6], dev[:, 6:9], dev[:, 9]

    def get_rays(self, iteration: int):
        cfg = self.config
        if cfg.use_preprocessed_data:
            if self._batch_iter is None or iteration % len(self.train_dataloader) == 0:
                self._batch_iter = iter(self.train_dataloader)
            rays, rgbs, idxs = next(self._batch_iter)
            return self._to_device(rays, rgbs, idxs)
        if cfg.get("add_upsample", -1) > 0 and iteration == cfg.add_upsample:
            cfg.downsample_train = max(cfg.downsample_train / 2, 1)
            self.train_dataset, self.test_dataset = prep_dataset(self.enable_lpips, cfg)
            self.allrays, self.allrgbs, self.allidxs, self.trainingsampler = prep_sampler(
                self.enable_lpips, cfg, self.train_dataset)
        if cfg.get("add_lpips", -1) > 0 and iteration == cfg.add_lpips:
            self.enable_lpips = True
            self.train_dataset, self.test_dataset = prep_dataset(True, cfg)
            self.allrays, self.allrgbs, self.allidxs, self.trainingsampler = prep_sampler(True, cfg, self.train_dataset)
        ids = self.trainingsampler.nextids()
        replicas, dp_rank = self._replica()
        if replicas > 1 and not self.enable_lpips:
            ids = torch.chunk(ids, replicas, dim=0)[dp_rank]
        return self._to_device(self.allrays[ids], self.allrgbs[ids], self.allidxs[ids])

    # -- Gaussian ----------------------------------------------------------------------------
    def _init_gaussian(self):
        cfg = self.config
        self.test_dataset = prep_testdataset_gs(cfg)
        self.distributed_sampler = None
        if cfg.is_train:
            self.train_dataset = prep_traindataset_gs(cfg)
            self.full_train_dataset = self.train_dataset
            if cfg.train_all_data:
                self.train_dataset = ConcatDataset([self.train_dataset, self.test_dataset])
            self._build_train_loader()
        self.test_loader = DataLoader(self.test_dataset, batch_size=1, collate_fn=self.test_dataset.collate_fn,
                                      shuffle=False, num_workers=0)
        self.test_loader_iter = iter(self.test_loader)
        self.white_bg = self.test_dataset.white_bg
        self.test_data_size = len(self.test_dataset)

    def _build_train_loader(self):
        cfg = self.config
        ddp = bool(cfg.get("DDP", False)) and torch.distributed.is_initialized()
        self.distributed_sampler = CameraDistributedSampler(self.train_dataset) if ddp else None
        collate = getattr(self.train_dataset, "collate_fn", None) or self.full_train_dataset.collate_fn
        self.train_loader = DataLoader(self.train_dataset, batch_size=1, collate_fn=collate, shuffle=not ddp,
                                       num_workers=0, sampler=self.distributed_sampler)
        self.train_loader_iter = iter(self.train_loader)
        self.train_data_size = len(self.train_dataset)

    def get_camera(self, split: str = "train"):
        if self.config.max_iter_each_block != -1 and split == "train":
            self.iter_cnt += 1
            assert self.iter_cnt <= self.config.max_iter_each_block, \
                "exceeded the iteration budget of the current block; switch to the next block"
        attr = "train_loader_iter" if split == "train" else "test_loader_iter"
        loader = self.train_loader if split == "train" else self.test_loader
        try:
            return next(getattr(self, attr))
        except StopIteration:
            setattr(self, attr, iter(loader))
            return next(getattr(self, attr))

    # -- spatial cells for dynamic (block-wise) Gaussian training --------------------------------
    def divide_dataset(self, plane_division, aabb_xy):
        """Assign each training camera to the XY cell under its centre; returns cells' camera counts."""
        nx, ny = plane_division
        self._cells_ny = int(ny)
        (x0, y0), (x1, y1) = aabb_xy
        self.cells = [[] for _ in range(nx * ny)]
        for i, cam in enumerate(self.full_train_dataset.cameras):
            c = cam.camera_center
            bx = min(max(int((float(c[0]) - x0) / (x1 - x0) * nx), 0), nx - 1)
            by = min(max(int((float(c[1]) - y0) / (y1 - y0) * ny), 0), ny - 1)
            self.cells[bx * ny + by].append(i)
        return [len(c) for c in self.cells]

    def switch_cell(self, cell_idx):
        """``cell_idx``: row-major cell index, or the reference's ``(bx, by)`` block coordinate."""
        if not isinstance(cell_idx, int):
            bx, by = (int(v) for v in cell_idx)
            cell_idx = bx * int(self._cells_ny) + by
        self.iter_cnt = 0
        n_scales = len(getattr(self.full_train_dataset, "resolution_scales", [1.0]))
        items = [c * n_scales + k for c in self.cells[cell_idx] for k in range(n_scales)]    # every scale of the cell's cameras
        self.train_dataset = torch.utils.data.Subset(self.full_train_dataset, items)
        self._build_train_loader()

    def use_all_data(self):
        self.iter_cnt = 0
        self.train_dataset = self.full_train_dataset
        self._build_train_loader()

"""Octree-GS encoding: Scaffold-GS anchors organised in levels of detail (reference:
landmark/nerf_components/model_components/fields/encodings/octreegs_encoding.py:30-1101).

Every anchor carries an integer ``level`` (voxel size ``voxel_size / fork^level``) and a float
``extra_level``.  Per view, :meth:`set_anchor_mask` keeps anchors whose level does not exceed the level
predicted from the camera distance; training can open levels progressively (coarse to fine).
The PLY stores ``level``, ``extra_level`` and ``info`` (voxel size, standard distance) next to the
Scaffold-GS properties.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int
from typing import Dict

import numpy as np
import torch
from torch import nn

from ....ops import native
from ....ops.knn import distCUDA2
from ...utils.ply_utils import read_ply, write_ply
from .scaffoldgs_encoding import ScaffoldGSEncoding, segment_amax, voxel_keys

P = native.P
native.register_signature("lmb_octree_lod_mask", [c_int, P, P, P, c_float, c_float, c_float, c_float, c_float, c_float,
                                                   c_float, c_int, c_int, P, P, P, P])
_MODES = {"floor": 0, "round": 1, "ceil": 2, "progressive": 3}


class OctreeGSEncoding(ScaffoldGSEncoding):
    def __init__(self, feat_dim: int = 32, n_offsets: int = 10, fork: int = 2, visible_threshold: float = -1,
                 dist2level: str = "round", base_layer: int = 10, progressive: bool = True, extend: float = 1.1,
                 percent_dense: float = 0.01, enable_lod: bool = True, device="cuda"):
        super().__init__(feat_dim=feat_dim, n_offsets=n_offsets, voxel_size=0.0, percent_dense=percent_dense,
                         device=device)
        assert dist2level in _MODES, f"Unknown dist2level: {dist2level}"
        self.fork, self.visible_threshold, self.dist2level = fork, visible_threshold, dist2level
        self.base_layer, self.progressive, self.extend, self.enable_lod = base_layer, progressive, extend, enable_lod
        self.levels, self.init_level, self.standard_dist = 1, 0, 1.0
        self.coarse_intervals = []
        self.init_pos = torch.zeros(3, device=self.device)
        self.cam_infos = torch.empty(0, 4, device=self.device)
        self._level = nn.Parameter(torch.zeros(0, 1, device=self.device), requires_grad=False)
        self._extra_level = nn.Parameter(torch.zeros(0, device=self.device), requires_grad=False)
        self._anchor_mask = torch.ones(0, dtype=torch.bool, device=self.device)
        self._prog_ratio = None
        self.transition_mask = None
        self.save_init_kwargs(locals())

    @property
    def get_level(self):
        return self._level

    @property
    def get_extra_level(self):
        return self._extra_level

    # -- level bookkeeping ------------------------------------------------------------------------------
    def set_coarse_interval(self, coarse_iter: int, coarse_factor: float):
        """Iterations at which the next finer level opens: a geometric series summing to ``coarse_iter``."""
        self.coarse_intervals = []
        n = self.levels - 1 - self.init_level
        if n > 0:
            q = 1.0 / coarse_factor
            a1 = coarse_iter * (1 - q) / (1 - q ** n) if abs(1 - q ** n) > 1e-12 else coarse_iter / n
            acc = 0.0
            for i in range(n):
                acc += a1 * q ** i
                self.coarse_intervals.append(acc)

    @torch.no_grad()
    def set_level(self, points, cameras, scales, dist_ratio: float = 0.95, init_level: int = -1, levels: int = -1):
        """Number of levels from the spread of camera-to-point distances (quantiles ``dist_ratio``)."""
        points = points.to(self.device)
        infos, dists = [], []
        for scale in scales:
            for cam in cameras:
                if getattr(cam, "resolution_scale", 1.0) != scale:
                    continue
                c = cam.camera_center.float().to(self.device)
                infos.append(torch.cat((c, torch.tensor([scale], device=self.device))))
                d = (points - c).norm(dim=1)
                dists.append(torch.stack((torch.quantile(d, 1 - dist_ratio), torch.quantile(d, dist_ratio))) * scale)
        self.cam_infos = torch.stack(infos)
        all_dist = torch.cat(dists)
        dist_max, dist_min = torch.quantile(all_dist, dist_ratio), torch.quantile(all_dist, 1 - dist_ratio)
        self.standard_dist = float(dist_max)
        self.levels = levels if levels != -1 else int(torch.round(torch.log2(dist_max / dist_min) / math.log2(self.fork))) + 1
        self.levels = max(self.levels, 1)
        self.init_level = init_level if init_level != -1 else int(self.levels / 2)

    def map_to_int_level(self, pred_level: torch.Tensor, cur_level: int, levels: torch.Tensor = None) -> torch.Tensor:
        if self.dist2level == "progressive":
            pred = torch.clamp(pred_level + 1.0, min=0.9999, max=cur_level + 0.9999)
            int_level = torch.floor(pred).int()
            if levels is not None:
                self._prog_ratio = torch.frac(pred).unsqueeze(1)
                self.transition_mask = levels.squeeze(1).int() == int_level
            return int_level
        fn = {"floor": torch.floor, "round": torch.round, "ceil": torch.ceil}[self.dist2level]
        return torch.clamp(fn(pred_level).int(), min=0, max=cur_level)

    def octree_sample(self, data: torch.Tensor, init_pos: torch.Tensor):
        positions, levels = [], []
        for cur_level in range(self.levels):
            cur_size = self.voxel_size / (float(self.fork) ** cur_level)
            pos = torch.unique(torch.round((data - init_pos) / cur_size), dim=0) * cur_size + init_pos
            positions.append(pos)
            levels.append(torch.full((pos.shape[0],), cur_level, dtype=torch.int32, device=self.device))
        return torch.cat(positions), torch.cat(levels)

    @torch.no_grad()
    def weed_out(self, positions: torch.Tensor, levels: torch.Tensor):
        """Drop voxels that (averaged over the training cameras) are rarely selected by the LOD rule."""
        if self.cam_infos.shape[0] == 0 or positions.shape[0] == 0:
            keep = torch.ones(positions.shape[0], dtype=torch.bool, device=positions.device)
            return positions, levels, 0.0, keep
        count = torch.zeros(positions.shape[0], device=self.device)
        for cam in self.cam_infos:
            dist = (positions - cam[:3]).norm(dim=1) * cam[3]
            pred = torch.log2(self.standard_dist / dist) / math.log2(self.fork)
            count += (levels <= self.map_to_int_level(pred, self.levels - 1)).float()
        count /= self.cam_infos.shape[0]
        keep = count > self.visible_threshold
        return positions[keep], levels[keep], float(count.mean()), keep

    def create_from_pcd(self, pcd, spatial_lr_scale: float = 1.0):
        pts = torch.as_tensor(np.asarray(pcd.points), dtype=torch.float32, device=self.device)
        box_min, box_max = float(pts.min()) * self.extend, float(pts.max()) * self.extend
        if box_min > 0:
            box_min = float(pts.min()) / self.extend
        box_d = box_max - box_min
        if self.base_layer < 0:
            d = distCUDA2(pts)
            median = float(torch.kthvalue(d, max(int(d.shape[0] * 0.5), 1)).values)
            self.base_layer = int(math.log2(box_d / max(median, 1e-9))) - self.levels + 1
        self.voxel_size = box_d / (float(self.fork) ** self.base_layer)
        self.init_pos = torch.tensor([box_min] * 3, device=self.device)
        positions, levels = self.octree_sample(pts, self.init_pos)
        if self.visible_threshold < 0:
            self.visible_threshold = 0.0
            positions, levels, self.visible_threshold, _ = self.weed_out(positions, levels)
        positions, levels, _, _ = self.weed_out(positions, levels)
        self._init_from_positions(positions)
        self._level = nn.Parameter(levels.float()[:, None], requires_grad=False)
        self._extra_level = nn.Parameter(torch.zeros(positions.shape[0], device=self.device), requires_grad=False)
        self._anchor_mask = torch.ones(positions.shape[0], dtype=torch.bool, device=self.device)

    # -- LOD selection ----------------------------------------------------------------------------------------
    @torch.no_grad()
    def set_anchor_mask(self, cam_center, iteration: int, resolution_scale: float, mlp_is_training: bool = True):
        n = self._anchor.shape[0]
        if not self.enable_lod or n == 0:
            self._anchor_mask = torch.ones(n, dtype=torch.bool, device=self.device)
            return
        if self.progressive and mlp_is_training:
            coarse_index = int(np.searchsorted(self.coarse_intervals, iteration)) + 1 + self.init_level
        else:
            coarse_index = int(self._level.max() - self._level.min()) + 1
        cam_center = cam_center.to(self.device).float()
        if self._anchor.is_cuda:
            mask = torch.empty(n, dtype=torch.uint8, device=self.device)
            prog = self.dist2level == "progressive"
            ratio = torch.empty(n, device=self.device) if prog else None
            trans = torch.empty(n, dtype=torch.uint8, device=self.device) if prog else None
            c = cam_center.tolist()
            native.check(native.lib().lmb_octree_lod_mask(
                n, self._anchor.data_ptr(), self._level.data_ptr(), self._extra_level.data_ptr(), c[0], c[1], c[2],
                self.voxel_size / 2, float(self.fork), float(self.standard_dist), float(resolution_scale),
                coarse_index - 1, _MODES[self.dist2level], mask.data_ptr(), native.ptr(ratio), native.ptr(trans),
                native.stream_ptr()), "octree_lod_mask")
            self._anchor_mask = mask.bool()
            if prog:
                self._prog_ratio, self.transition_mask = ratio[:, None], trans.bool()
            return
        pos = self._anchor + (self.voxel_size / 2) / (float(self.fork) ** self._level)
        dist = (pos - cam_center).norm(dim=1) * resolution_scale
        pred = torch.log2(self.standard_dist / dist) / math.log2(self.fork) + self._extra_level
        self._anchor_mask = self._level.squeeze(1) <= self.map_to_int_level(pred, coarse_index - 1, self._level)

    def plot_levels(self):
        """Print and return ``[(level, anchors, share of all anchors)]`` (reference: octreegs_encoding.py:1086-1101)."""
        level = self._level.detach().squeeze(1)
        total = max(int(level.shape[0]), 1)
        rows = []
        for lv in range(int(self.levels)):
            n = int((level == lv).sum())
            rows.append((lv, n, n / total))
            print(f"Level {lv}: {n}, Ratio: {n / total}")
        return rows

    def get_remove_duplicates(self, grid_coords: torch.Tensor, selected_grid_coords_unique: torch.Tensor,
                              use_chunk: bool = True) -> torch.Tensor:
        """``[N]`` mask of the rows of ``grid_coords`` that also appear in ``selected_grid_coords_unique`` (integer
        voxel coordinates): one packed 64-bit key per voxel and a sorted membership test instead of the reference's
        chunked all-pairs comparison (octreegs_encoding.py:628-660); ``use_chunk`` is accepted for compatibility."""
        return torch.isin(voxel_keys(torch.round(grid_coords)), voxel_keys(torch.round(selected_grid_coords_unique)))

    def construct_list_of_attributes(self):
        return super().construct_list_of_attributes() + ["level", "extra_level", "info"]

    # -- PLY ---------------------------------------------------------------------------------------------------
    def save_ply(self, path: str):
        cols = self._ply_columns()
        n = self._anchor.shape[0]
        cols["level"] = self._level.detach().cpu().numpy()[:, 0].astype(np.float32)
        cols["extra_level"] = self._extra_level.detach().cpu().numpy().astype(np.float32)
        info = np.zeros(n, dtype=np.float32)
        if n >= 2:
            info[0], info[1] = self.voxel_size, self.standard_dist
        cols["info"] = info
        write_ply(path, cols, comments=[f"voxel_size {self.voxel_size}", f"standard_dist {self.standard_dist}",
                                        f"levels {self.levels}", f"init_pos {float(self.init_pos[0])}"])

    def load_ply_to_state_dict(self, path: str, map_location="cpu") -> Dict[str, torch.Tensor]:
        state = super().load_ply_to_state_dict(path, map_location)
        v = read_ply(path)
        state["_level"] = torch.from_numpy(np.asarray(v["level"], np.float32)[:, None].copy()).to(map_location)
        state["_extra_level"] = torch.from_numpy(np.asarray(v["extra_level"], np.float32).copy()).to(map_location)
        info = np.asarray(v["info"], np.float32)
        if len(info) >= 2:
            state["_info"] = torch.tensor([float(info[0]), float(info[1])])
        return state

    def load_encoding_state(self, state):
        super().load_encoding_state(state)
        n = self._anchor.shape[0]
        lvl = state.get("_level", torch.zeros(n, 1))
        self._level = nn.Parameter(lvl.to(self.device).float().reshape(n, 1), requires_grad=False)
        self._extra_level = nn.Parameter(state.get("_extra_level", torch.zeros(n)).to(self.device).float().reshape(n),
                                         requires_grad=False)
        if "_info" in state:
            self.voxel_size, self.standard_dist = float(state["_info"][0]), float(state["_info"][1])
        self.levels = int(self._level.max()) + 1 if n else 1
        self._anchor_mask = torch.ones(n, dtype=torch.bool, device=self.device)

    # -- structural updates -------------------------------------------------------------------------------------------
    def prune_anchor(self, mask, optimizer):
        super().prune_anchor(mask, optimizer)
        self._level = nn.Parameter(self._level[~mask], requires_grad=False)
        self._extra_level = nn.Parameter(self._extra_level[~mask], requires_grad=False)

    def _fresh_voxels(self, xyz, size, level_anchors, level):
        """Unique voxel centres of ``xyz`` at ``size`` that hold no anchor of this level yet and pass the
        visibility test; returns ``(centres, keep-mask over unique voxels, inverse indices)``."""
        if xyz.shape[0] == 0:
            e = torch.zeros(0, dtype=torch.bool, device=self.device)
            return torch.zeros(0, 3, device=self.device), e, torch.zeros(0, dtype=torch.long, device=self.device)
        uniq, inverse = torch.unique(torch.round((xyz - self.init_pos) / size), return_inverse=True, dim=0)
        occupied = voxel_keys(torch.round((level_anchors - self.init_pos) / size))
        keep = ~torch.isin(voxel_keys(uniq), occupied)
        centres = uniq[keep] * size + self.init_pos
        lv = torch.full((centres.shape[0],), level, dtype=torch.int32, device=self.device)
        centres, _, _, weed = self.weed_out(centres, lv)
        k2 = keep.clone()
        k2[keep] = weed
        return centres, k2, inverse

    @torch.no_grad()
    def anchor_growing(self, iteration, grads, threshold, update_ratio, extra_ratio, extra_up, offset_mask, optimizer):
        k = self.n_offsets
        init_n = self._anchor.shape[0]
        grads = grads.clone()
        grads[~offset_mask] = 0.0
        anchor_grads = grads.view(-1, k).sum(-1) / (offset_mask.view(-1, k).sum(-1) + 1e-6)
        finished_coarse = (not self.progressive) or (not self.coarse_intervals) or iteration > self.coarse_intervals[-1]
        update_value = self.fork ** update_ratio
        for cur_level in range(self.levels):
            level_mask = (self._level.squeeze(1) == cur_level)
            if level_mask.sum() == 0:
                continue
            cur_size = self.voxel_size / (float(self.fork) ** cur_level)
            cur_thr = threshold * (update_value ** cur_level)
            ds_size, ds_thr = cur_size / self.fork, cur_thr * update_value
            cand = (grads >= cur_thr) & (grads < ds_thr)
            cand_ds = grads >= ds_thr
            cand_extra = anchor_grads >= cur_thr * extra_ratio
            inc = self._anchor.shape[0] - init_n
            if inc > 0:
                zk = torch.zeros(inc * k, dtype=torch.bool, device=self.device)
                cand, cand_ds = torch.cat((cand, zk)), torch.cat((cand_ds, zk))
                cand_extra = torch.cat((cand_extra, torch.zeros(inc, dtype=torch.bool, device=self.device)))
            rep = level_mask[:, None].expand(-1, k).reshape(-1)
            cand, cand_ds = cand & rep, cand_ds & rep
            if finished_coarse:
                self._extra_level.data += extra_up * cand_extra.float()
            all_xyz = (self._anchor[:, None] + self._offset * self.get_scaling[:, None, :3]).view(-1, 3)
            level_anchors = self._anchor[level_mask]
            centres, keep, inverse = self._fresh_voxels(all_xyz[cand], cur_size, level_anchors, cur_level)
            if finished_coarse and cur_level < self.levels - 1:
                centres_ds, _, _ = self._fresh_voxels(all_xyz[cand_ds], ds_size, level_anchors, cur_level + 1)
            else:
                centres_ds = torch.zeros(0, 3, device=self.device)
            if centres.shape[0] + centres_ds.shape[0] == 0:
                continue
            if centres.shape[0] > 0:
                feats = self._anchor_feat[:, None].expand(-1, k, -1).reshape(-1, self.feat_dim)[cand]
                new_feat = segment_amax(feats, inverse, keep.shape[0])[keep]
            else:
                new_feat = torch.zeros(0, self.feat_dim, device=self.device)
            a = self._new_anchor_tensors(centres, cur_size, new_feat)
            b = self._new_anchor_tensors(centres_ds, ds_size, torch.zeros(centres_ds.shape[0], self.feat_dim, device=self.device))
            new = {key: torch.cat((a[key], b[key]), 0) for key in a}
            new_level = torch.cat((torch.full((centres.shape[0], 1), float(cur_level), device=self.device),
                                   torch.full((centres_ds.shape[0], 1), float(cur_level + 1), device=self.device)))
            self._append(new, optimizer)
            self._level = nn.Parameter(torch.cat((self._level, new_level), 0), requires_grad=False)
            self._extra_level = nn.Parameter(torch.cat((self._extra_level, torch.zeros(new_level.shape[0], device=self.device))),
                                             requires_grad=False)

    @torch.no_grad()
    def adjust_anchor(self, iteration=0, check_interval=100, success_threshold=0.8, grad_threshold=0.0002,
                      update_ratio=0.5, extra_ratio=4.0, extra_up=0.25, min_opacity=0.005, optimizer=None):
        grads = self.offset_gradient_accum / self.offset_denom
        grads[grads.isnan()] = 0.0
        offset_mask = (self.offset_denom > check_interval * success_threshold * 0.5).squeeze(1)
        self.anchor_growing(iteration, torch.norm(grads, dim=-1), grad_threshold, update_ratio, extra_ratio, extra_up,
                            offset_mask, optimizer)
        self._after_growing(offset_mask)
        self._prune_by_opacity(check_interval, success_threshold, min_opacity, optimizer)
        self._anchor_mask = torch.ones(self._anchor.shape[0], dtype=torch.bool, device=self.device)

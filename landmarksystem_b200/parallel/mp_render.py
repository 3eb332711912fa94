"""Model-parallel rendering by spatial blocks.

Each rank holds the grids of a rectangular window of scene blocks (what dynamic loading keeps resident on that
GPU) and renders, for every ray, only the segment that crosses its window; the per-rank records (colour,
transmittance, depth, opacity, entry distance) are then merged front to back across the ranks by ONE kernel per
rank that pulls the peers' records over NVLink, orders them by entry distance, composites them and stores the
finished pixels (``ops/csrc/fused_comm.cu: composite_merge_p2p_kernel``).  The reference has no counterpart: its
engine forbids model parallelism together with dynamic loading and only gathers data-parallel ray slices
(landmark/__init__.py:51-54, landmark/render/parallel_module/parallel_module.py:105-135)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .composite_merge import CompositeMerger, merge_reference


def block_window_of(part: int, parts: int, nx: int, ny: int):
    """Rectangular window of scene blocks kept by rank ``part`` of ``parts``: the ``nx x ny`` block lattice is cut into
    ``px x py = parts`` equal rectangles, rows first (``px`` is the largest divisor of ``parts`` that also divides
    ``nx``).  Returns ``(row0, col0, rows, cols)``."""
    px = max(d for d in range(1, parts + 1) if parts % d == 0 and nx % d == 0)
    py = parts // px
    assert ny % py == 0, f"a {nx} x {ny} block lattice cannot be cut into {parts} equal rectangles"
    rows, cols = nx // px, ny // py
    return (part // py) * rows, (part % py) * cols, rows, cols


def slice_model_to_block_window(model, part: int, parts: int):
    """Keep only the ``part``-th of ``parts`` equal rectangles of the model's spatial blocks (blocks are ordered
    ``bx * ny + by``): the grids of every plane/line encoding are sliced and the scene manager's resident window is set
    accordingly, so lookups outside the window return "no data".  Returns ``(first_block, n_blocks)``."""
    sm = model.scene_manager
    nx, ny = sm._partition
    row0, col0, rows, cols = block_window_of(part, parts, nx, ny)
    keep = torch.tensor([(row0 + r) * ny + (col0 + c) for r in range(rows) for c in range(cols)], dtype=torch.long)
    for enc in model.modules():
        planes, lines = getattr(enc, "plane_coef", None), getattr(enc, "line_coef", None)
        if planes is None or lines is None:
            continue
        for plist in (planes, lines):
            for p in plist:
                if p.shape[0] == nx * ny:
                    p.data = p.data.index_select(0, keep.to(p.device)).contiguous()
        if getattr(enc, "use_shadow", False):
            enc.enable_shadow(False)
    sm.assign_local_block_partition([rows, cols])
    sm.assign_relative_block_idx(row0 * ny + col0)
    return row0 * ny + col0, rows * cols


class ModelParallelRenderer:
    """``model`` must offer ``render_partial(rays, N_samples) -> [R, 8]`` (see ``GridNeRF.render_partial``)."""

    def __init__(self, model, max_rays: int, group=None, white_bg: Optional[bool] = None):
        self.model = model
        if white_bg is None:                              # follow the model's own renderer
            white_bg = bool(getattr(getattr(model, "renderer", None), "white_bg", False))
        self.bg = 1.0 if white_bg else 0.0
        self.group = group
        self.merger: Optional[CompositeMerger] = None
        self.max_rays = int(max_rays)

    @torch.no_grad()
    def render(self, rays: torch.Tensor, N_samples: int = -1, root: int = -1, chunk: Optional[int] = None
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``(rgb [R,3] in [0,1], depth [R], opacity [R])`` on ``root`` (every rank when ``root == -1``)."""
        R = rays.shape[0]
        chunk = chunk or R
        partial = torch.cat([self.model.render_partial(rays[s:s + chunk], N_samples) for s in range(0, R, chunk)])
        if rays.is_cuda and torch.distributed.is_initialized() and torch.distributed.get_world_size(self.group) > 1:
            if self.merger is None or self.merger.max_rays < R:
                self.merger = CompositeMerger(max(R, self.max_rays), self.group)
            out = self.merger.merge(partial, bg=self.bg, root=root).clone()
        else:                                            # one rank (or CPU): the same merge in PyTorch
            out = merge_reference(partial[None], bg=self.bg)
        return out[:, :3].clamp(0.0, 1.0), out[:, 4], out[:, 5]

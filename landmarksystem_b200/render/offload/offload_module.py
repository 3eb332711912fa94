"""Dynamic loading wrapper: keeps only a window of spatial blocks on the device and streams the next
window in while the camera moves (reference: landmark/render/parameter_loader/offload_module.py:14-138).

Configuration (``inference_config.offload_config``): ``local_plane_split`` (window size in blocks),
``plane_split`` (scene partition), ``use_nccl``, ``use_h2d``, ``channel_last`` (accepted; the native
layout already is channels-last), ``sync_switch``; additions: ``dtype`` ("bf16" halves the streamed
bytes, the lookup kernels read bf16 directly), ``swap_delay`` (frames between issuing and swapping) and
``prefetch_frames`` (how many frames ahead of the camera the window is chosen, see ``_pre_forward``).

The reference starts loading a window when the camera has already crossed into a new block
(landmark/render/parameter_loader/offload_module.py:98-123).  Here the camera track is extrapolated: the window is
centred on the block the camera will be over ``prefetch_frames`` frames from now (velocity = smoothed displacement
per frame), so the copy is issued before the boundary is reached and the swap has happened by the time the camera
arrives.  ``stats()`` reports how many frames found the camera's block missing from the resident window (a stall:
the frame then waits for the copy) and how many swaps had to wait for an unfinished copy."""
from __future__ import annotations

from typing import Any, Mapping

import torch
from torch import nn

from ...utils import Config
from ..inference_module import InferenceModule
from .block import create_blocks
from .buffer_manager import BufferManager
from .utils import calculate_block_neighbours, mergeable_keys


def _find_state_dict(state):
    return state["state_dict"] if "state_dict" in state else state


def _owner(model: nn.Module, key: str):
    """``(module, key relative to it)`` of the deepest module on the path of ``key`` that knows how to
    convert checkpoint slices (defines ``block_to_internal``); the root model if none does."""
    parts = key.split(".")
    mod, best, best_depth = model, model, 0
    for i, p in enumerate(parts[:-1]):
        try:
            child = mod[int(p)] if p.isdigit() else getattr(mod, p)
        except (AttributeError, IndexError, KeyError, TypeError):
            break
        if not isinstance(child, nn.Module):
            break
        mod = child
        if hasattr(mod, "block_to_internal"):
            best, best_depth = mod, i + 1
    return best, parts[best_depth:]


class OffloadModule(nn.Module):
    def __init__(self, model, merged_state_dict, config: Config, device="cuda"):
        super().__init__()
        self.model = model
        self.inner = model.inter_model if isinstance(model, InferenceModule) else model
        self.scene_mgr = model.scene_manager if isinstance(model, InferenceModule) else getattr(model, "scene_manager")
        self.device = torch.device(device)
        if isinstance(config.get("plane_split"), (list, tuple)):
            self.scene_mgr.assign_block_partition(config.plane_split)
        self.scene_mgr.assign_local_block_partition(config.local_plane_split)
        plane_split = [int(v) for v in self.scene_mgr.block_partition]
        use_nccl = bool(config.get("use_nccl", False))
        group, use_h2d = None, True
        if use_nccl and torch.distributed.is_initialized():
            from ...comm import CommContext, ParallelMode

            ctx = CommContext()
            if ctx.is_initialized():
                group = ctx.get_group(ParallelMode.DYNAMIC_LOAD)
                use_h2d = ctx.get_local_rank(ParallelMode.DYNAMIC_LOAD) == 0
        use_h2d = bool(config.get("use_h2d", use_h2d))
        fanout = bool(config.get("fanout", True)) and group is not None and self.device.type == "cuda"
        if config.get("channel_last", False) and hasattr(self.inner, "channel_last"):
            self.inner.channel_last()
        dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, None: None, "fp32": None}[config.get("dtype")]
        merged = {k: self._to_reference(k, v) for k, v in _find_state_dict(merged_state_dict).items()}
        self.merge_config = self.inner.get_merge_config()
        self.streamed = mergeable_keys(self.merge_config, merged)
        blocks = create_blocks(self.merge_config, merged, plane_split, to_internal=self._to_internal, dtype=dtype,
                               pin_memory=self.device.type == "cuda")
        self.buffer_manager = BufferManager(blocks, plane_split, config.local_plane_split, self.device, use_nccl, use_h2d,
                                            group, int(config.get("swap_delay", 0 if group is None else 4)), fanout=fanout)
        # everything that is not streamed is loaded once, the streamed parameters start empty
        rest = {k: v for k, v in merged.items() if k not in self.streamed}
        self.model.load_from_state_dict(rest, False)
        self._shrink_streamed_params()
        self.init = True
        self.prefetch_frames = int(config.get("prefetch_frames", 8))
        self._last_xy = None
        self._velocity = None
        self.frames = self.stalled_frames = self.late_swaps = 0

    # -- layout glue --------------------------------------------------------------------------------------
    def _to_internal(self, key: str, piece: torch.Tensor) -> torch.Tensor:
        mod, tail = _owner(self.inner, key)
        fn = getattr(mod, "block_to_internal", None)
        return fn(".".join(tail), piece) if fn is not None else piece

    def _to_reference(self, key: str, tensor: torch.Tensor) -> torch.Tensor:
        """Checkpoint variants (channels-last planes) brought to the layout the merge configuration describes."""
        try:
            mod, tail = _owner(self.inner, key)
        except (AttributeError, IndexError, KeyError):
            return tensor
        fn = getattr(mod, "to_reference_layout", None)
        return fn(".".join(tail), tensor) if fn is not None and torch.is_tensor(tensor) else tensor

    def _targets(self):
        """``{buffer key: [(module, attribute name or list index, slot or None)]}`` the buffer tensors feed."""
        out = {}
        for key in self.buffer_manager.get_buffer().state_dict:
            if "{}" in key:
                n = self.buffer_manager.get_buffer().n_slots
                out[key] = [(key.replace("{}", str(s)), s) for s in range(n)]
            else:
                out[key] = [(key, None)]
        return out

    def _set_param(self, name: str, tensor: torch.Tensor):
        parts = name.split(".")
        mod = self.inner
        for p in parts[:-1]:
            mod = mod[int(p)] if p.isdigit() else getattr(mod, p)
        leaf = parts[-1]
        holder = mod[int(leaf)] if leaf.isdigit() else getattr(mod, leaf)
        if isinstance(holder, nn.Parameter):
            holder.data = tensor
            holder.requires_grad_(False)
        else:
            setattr(mod, leaf, tensor)

    def _shrink_streamed_params(self):
        for name in self.streamed:
            try:
                self._set_param(name, torch.empty(0, device=self.device))
            except (AttributeError, IndexError, KeyError):
                pass

    def load_buffer(self):
        buf = self.buffer_manager.get_buffer()
        for key, targets in self._targets().items():
            for name, slot in targets:
                t = buf.state_dict[key] if slot is None else buf.state_dict[key][slot]
                try:
                    self._set_param(name, t)
                except (AttributeError, IndexError, KeyError):
                    pass
        self.scene_mgr.assign_relative_block_idx(buf.local_block_idxes[0])

    def __getattr__(self, item):
        try:
            return super().__getattr__(item)
        except AttributeError:
            return getattr(super().__getattr__("model"), item)

    def load_from_state_dict(self, state_dict: Mapping[str, Any], strict: bool = False):
        rest = {k: v for k, v in _find_state_dict(state_dict).items() if k not in self.streamed}
        return self.model.load_from_state_dict(rest, False)

    # -- per-frame hook ---------------------------------------------------------------------------------------
    def _block_at(self, xy) -> int:
        sm = self.scene_mgr
        nx, ny = sm._partition
        lo = sm.aabb[0, :2].tolist()
        width = sm.block_width.tolist()
        bx = min(max(int((xy[0] - lo[0]) // width[0]), 0), nx - 1)
        by = min(max(int((xy[1] - lo[1]) // width[1]), 0), ny - 1)
        return bx * ny + by

    def _window_of(self, block: int):
        return calculate_block_neighbours(block, self.scene_mgr.block_partition.tolist(), self.scene_mgr.local_block_partition)

    def _predicted_block(self, xy):
        """Block under the camera ``prefetch_frames`` frames ahead, from an exponentially smoothed per-frame velocity."""
        if self._last_xy is not None:
            step = (xy[0] - self._last_xy[0], xy[1] - self._last_xy[1])
            self._velocity = step if self._velocity is None else tuple(0.5 * v + 0.5 * s for v, s in zip(self._velocity, step))
        self._last_xy = xy
        if self._velocity is None or self.prefetch_frames <= 0:
            return self._block_at(xy)
        return self._block_at((xy[0] + self._velocity[0] * self.prefetch_frames, xy[1] + self._velocity[1] * self.prefetch_frames))

    def stats(self) -> dict:
        mgr = self.buffer_manager
        return {"frames": self.frames, "stalled_frames": self.stalled_frames, "late_swaps": self.late_swaps,
                "bytes_h2d": mgr.bytes_h2d, "bytes_d2d": mgr.bytes_d2d, "bytes_pushed": mgr.bytes_pushed}

    def _pre_forward(self, *args):
        rays = args[0]
        xy = [float(v) for v in (rays[0, :2] if torch.is_tensor(rays) else rays.data[0, :2]).tolist()]
        block_now = self._block_at(xy)
        mgr = self.buffer_manager
        self.frames += 1
        if self.init:
            self._predicted_block(xy)
            mgr.update_buffer(self._window_of(block_now), init=True)
            mgr.wait_update_done()
            self.load_buffer()
            self.init = False
            return
        target = self._window_of(self._predicted_block(xy))
        if block_now not in target:              # never trade the block under the camera for a predicted one
            target = self._window_of(block_now)
        mgr.update_buffer(target)
        if mgr.update_done():
            if not mgr.copy_finished():
                self.late_swaps += 1             # the swap frame arrived before the copy: this frame waits for it
            mgr.change_buffer()
            self.load_buffer()
        if block_now not in mgr.get_buffer().local_block_idxes:
            # the camera outran the stream (a jump, or a speed the window cannot follow): wait for data that covers it
            self.stalled_frames += 1
            if mgr.pending is None or block_now not in mgr.pending:
                if mgr.pending is not None:
                    mgr.change_buffer()
                mgr.update_buffer(self._window_of(block_now))
            mgr.change_buffer()
            self.load_buffer()

    def forward(self, *args, **kwargs):
        self._pre_forward(*args)
        return self.model(*args, **kwargs)

    def preprocess(self, *args, **kwargs):
        return self.model.preprocess(*args, **kwargs)

    def postprocess(self, *args, **kwargs):
        return self.model.postprocess(*args, **kwargs)

    def get_state_dict_from_ckpt(self, *a, **k):
        return self.model.get_state_dict_from_ckpt(*a, **k)

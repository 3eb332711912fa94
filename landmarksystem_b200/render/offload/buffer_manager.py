"""Streams scene blocks from pinned host memory into a double-buffered device window (reference:
landmark/render/parameter_loader/buffer_manager.py:19-122).

What differs by design:
* blocks that are already resident in the active window are copied device-to-device (HBM bandwidth)
  instead of being re-read over PCIe; only new blocks use ``cudaMemcpyAsync`` from pinned memory;
* the copies run on a side stream and are tracked by one CUDA event;
* ranks agree on the swap without a per-frame all-reduce: every rank issues the update on the same
  frame (same camera path) and swaps ``swap_delay`` frames later, waiting on its own event if the
  copy has not finished (the reference all-reduces a flag every frame while an update is in flight,
  buffer_manager.py:104);
* with several ranks per group and ``fanout`` (the default on CUDA) every rank reads 1/P of each new block from
  its own pinned copy over its own PCIe link and stores that piece into every peer's window over NVLink
  (``fused_comm.cu: fanout_push_kernel``, windows in peer-mapped memory, device-side barriers on the copy stream):
  the host link, which bounds streaming, is used P times in parallel.  Without ``fanout`` only the group leader reads
  the host and the others receive the window by a broadcast on the side stream, as in the reference
  (buffer_manager.py:68-80).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .block import Block
from .buffer import BUFFER_SIZE, Buffer, create_buffers


class BufferManager:
    def __init__(self, blocks: List[Block], plane_split: Sequence[int], local_plane_split: Sequence[int], device,
                 use_nccl: bool = False, use_h2d: bool = True, group=None, swap_delay: int = 0, fanout: bool = False):
        self.blocks, self.plane_split, self.local_plane_split = blocks, list(plane_split), list(local_plane_split)
        self.device = torch.device(device)
        self.use_nccl, self.use_h2d, self.group, self.swap_delay = use_nccl, use_h2d, group, int(swap_delay)
        self.cuda = self.device.type == "cuda"
        self.world = dist.get_world_size(group) if (dist.is_initialized() and group is not None) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.fanout = bool(fanout) and self.cuda and self.world > 1
        self.bytes_pushed = 0
        if self.fanout:
            from ctypes import c_int

            from ...comm.symmetric import PeerBarrier
            from ...ops import native

            native.register_signature("lmb_fanout_push", [native.P, native.P, native.P, native.P, c_int, c_int, c_int, native.P])
            self.use_h2d = True                       # every rank reads its share from its own pinned copy
            self.buffers = create_buffers(blocks, local_plane_split, self.device, BUFFER_SIZE, symmetric_group=group)
            self.barrier = PeerBarrier(group)
        else:
            self.buffers = create_buffers(blocks, local_plane_split, self.device, BUFFER_SIZE)
        self.active = 0
        self.copy_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.event: Optional[torch.cuda.Event] = None
        self.pending: Optional[List[int]] = None
        self.frames_since_issue = 0
        self.bytes_h2d = self.bytes_d2d = 0

    def get_buffer(self) -> Buffer:
        return self.buffers[self.active]

    FANOUT_MIN_BYTES = 1 << 16      # smaller tensors are read whole by every rank

    def _fill_fanout(self, target: Buffer, block_idxes: List[int]) -> None:
        """Resident blocks move device-to-device on every rank; of a new block each rank copies piece ``rank`` of
        every large tensor from its pinned host copy into its own window and pushes it to the peers."""
        import ctypes

        from ...ops import native

        current = self.get_buffer()
        resident = {b: s for s, b in enumerate(current.local_block_idxes)} if target is not current else {}
        offs, sizes = [], []
        for slot, b in enumerate(block_idxes):
            for key, dst in target.state_dict.items():
                if b in resident:
                    dst[slot].copy_(current.state_dict[key][resident[b]], non_blocking=True)
                    self.bytes_d2d += dst[slot].numel() * dst.element_size()
                    continue
                src = self.blocks[b].state_dict[key]
                nbytes = src.numel() * src.element_size()
                if nbytes < self.FANOUT_MIN_BYTES or nbytes % (16 * self.world) or not src.is_contiguous():
                    dst[slot].copy_(src.reshape(dst[slot].shape), non_blocking=True)
                    self.bytes_h2d += nbytes
                    continue
                piece = nbytes // self.world
                lo = self.rank * piece
                base = target.offsets[key] + slot * nbytes
                target.symm.local[base + lo: base + lo + piece].copy_(src.reshape(-1).view(torch.uint8)[lo: lo + piece],
                                                                      non_blocking=True)
                self.bytes_h2d += piece
                offs.append(base + lo)
                sizes.append(piece)
        target.local_block_idxes = list(block_idxes)
        if not offs:
            return
        # every rank has stopped reading this window (its copy stream waited for its render stream) before anyone stores
        # into it; after the second barrier every piece of every rank has landed
        self.barrier()
        arr = ctypes.c_longlong * len(offs)
        table = (ctypes.c_longlong * self.world)(*target.symm.peer_ptrs)
        native.check(native.lib().lmb_fanout_push(target.symm.local_ptr, table, arr(*offs), arr(*sizes), len(offs), self.rank, self.world,
                                                  native.stream_ptr()), "fanout_push")
        self.bytes_pushed += sum(sizes) * (self.world - 1)
        self.barrier()

    def _fill(self, target: Buffer, block_idxes: List[int]) -> None:
        if self.fanout:
            return self._fill_fanout(target, block_idxes)
        current = self.get_buffer()
        resident = {b: s for s, b in enumerate(current.local_block_idxes)} if target is not current else {}
        for slot, b in enumerate(block_idxes):
            for key, dst in target.state_dict.items():
                if b in resident:
                    dst[slot].copy_(current.state_dict[key][resident[b]], non_blocking=True)
                    self.bytes_d2d += dst[slot].numel() * dst.element_size()
                elif self.use_h2d:
                    src = self.blocks[b].state_dict[key]
                    dst[slot].copy_(src.reshape(dst[slot].shape), non_blocking=True)
                    self.bytes_h2d += src.numel() * src.element_size()
        if self.use_nccl and dist.is_initialized() and self.group is not None and dist.get_world_size(self.group) > 1:
            src_rank = dist.get_global_rank(self.group, 0)
            for dst in target.state_dict.values():
                dist.broadcast(dst, src=src_rank, group=self.group)
        target.local_block_idxes = list(block_idxes)

    def update_buffer(self, block_idxes: List[int], init: bool = False) -> bool:
        """Start loading the window ``block_idxes`` unless it is resident or already on its way."""
        if self.pending is not None:
            return False
        if not init and list(block_idxes) == self.get_buffer().local_block_idxes:
            return False
        target = self.buffers[self.active if init else self.active ^ 1]
        if self.cuda:
            self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))   # target is no longer read
            with torch.cuda.stream(self.copy_stream):
                self._fill(target, list(block_idxes))
                self.event = torch.cuda.Event()
                self.event.record(self.copy_stream)
        else:
            self._fill(target, list(block_idxes))
        self.pending = list(block_idxes)
        self.frames_since_issue = 0
        return True

    def wait_update_done(self) -> None:
        if self.cuda and self.event is not None:
            torch.cuda.current_stream(self.device).wait_event(self.event)
        self.pending = None

    def update_done(self) -> bool:
        """True when the pending window may be swapped in on this frame."""
        if self.pending is None:
            return False
        self.frames_since_issue += 1
        if self.swap_delay > 0:                       # deterministic swap frame, identical on every rank
            if self.frames_since_issue < self.swap_delay:
                return False
            self.wait_update_done_keep()
            return True
        return (not self.cuda) or self.event is None or self.event.query()

    def copy_finished(self) -> bool:
        """Whether the pending window's copies have completed on the device (always true on the CPU)."""
        return (not self.cuda) or self.event is None or self.event.query()

    def wait_update_done_keep(self) -> None:
        if self.cuda and self.event is not None:
            torch.cuda.current_stream(self.device).wait_event(self.event)

    def change_buffer(self) -> None:
        self.wait_update_done_keep()
        self.active ^= 1
        self.pending = None

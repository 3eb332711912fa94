"""Symmetric peer memory over NVLink: every rank allocates the same-sized buffer, the CUDA IPC handles
are exchanged once through ``torch.distributed`` and each rank maps all peers' buffers.  Kernels
then take an array of peer pointers and read / write remote HBM with ordinary loads and stores.

Also provides :class:`PeerBarrier`, a device-side barrier (release/acquire flags in peer memory, bounded
waits) that orders such kernels across GPUs without a host round trip or an NCCL call.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native

P = native.P
for _name, _sig in (("lmb_symm_alloc", [c_longlong, ctypes.POINTER(c_void_p)]), ("lmb_symm_free", [P]),
                    ("lmb_ipc_get_handle", [P, P]), ("lmb_ipc_open", [P, ctypes.POINTER(c_void_p)]),
                    ("lmb_ipc_close", [P]), ("lmb_peer_barrier", [P, P, c_int, c_int, P, P, c_longlong, P])):
    native.register_signature(_name, _sig)


def multicast_supported(device: int = 0) -> bool:
    """Whether the device reports NVLink multicast objects (what NVLS / ``multimem`` instructions need), read from the
    driver attribute only - nothing is allocated or bound.  The kernels of this package do not use multicast: their
    reduce-shaped traffic is either tiny or fused with an optimiser over plain peer loads, and a rank that dies while
    its memory is bound to a multicast object disturbs its peers' GPUs, which the rank-failure tests must avoid.  The
    probe lets a deployment log what the fabric offers (``NCCL_DEBUG=INFO`` shows whether NCCL uses it)."""
    if not torch.cuda.is_available():
        return False
    try:
        from cuda.bindings import driver as drv
    except ImportError:
        return False
    err, dev = drv.cuDeviceGet(int(device))
    if int(err) != 0:
        return False
    err, value = drv.cuDeviceGetAttribute(drv.CUdevice_attribute.CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev)
    return int(err) == 0 and bool(value)


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group``, each mapped into every other rank."""

    def __init__(self, nbytes: int, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.nbytes = int((nbytes + 255) // 256 * 256)
        lib = native.lib()
        ptr = c_void_p()
        native.check(lib.lmb_symm_alloc(self.nbytes, ctypes.byref(ptr)), "symm_alloc")
        self.local_ptr = ptr.value
        self.device = torch.device("cuda", torch.cuda.current_device())
        handle = (ctypes.c_ubyte * 64)()
        native.check(lib.lmb_ipc_get_handle(self.local_ptr, handle), "ipc_get_handle")
        handles: List[Optional[bytes]] = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        else:
            handles = [bytes(handle)]
        self.peer_ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            out = c_void_p()
            native.check(lib.lmb_ipc_open(buf, ctypes.byref(out)), "ipc_open")
            self.peer_ptrs.append(out.value)
            self._opened.append(out.value)
        self._keep = _RawCuda(self.local_ptr, self.nbytes)
        self.local = torch.as_tensor(self._keep, device=self.device)            # uint8 view of the local buffer
        self.ptr_table = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=self.device)

    def view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """Typed view of the local buffer starting at byte ``offset`` (must be suitably aligned)."""
        n = int(torch.tensor(shape).prod()) * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + n].view(dtype).view(*shape)

    def peer_table(self, offset: int = 0) -> torch.Tensor:
        """Device ``int64 [world]`` array of peer addresses of byte ``offset`` inside the buffer."""
        return self.ptr_table + offset

    def close(self):
        """Unmap the peers' buffers and free this rank's.  Safe only when no rank still uses the mappings: callers
        order it with a barrier across the group after synchronising their devices.  Idempotent.  There is deliberately
        no finaliser: garbage collection runs at different times on different ranks, and freeing memory that a peer's
        kernel may still address is worse than holding it until the process ends."""
        lib = native.lib()
        for p in self._opened:
            lib.lmb_ipc_close(p)
        self._opened = []
        if self.local_ptr:
            self.local = self._keep = None
            lib.lmb_symm_free(self.local_ptr)
            self.local_ptr = 0


class PeerBarrier:
    """Stream-ordered barrier across the ranks of a group, executed by a one-block kernel per rank."""

    def __init__(self, group=None, limit_cycles: int = 0):
        self.limit_cycles = int(limit_cycles)        # SM clocks a wait may last (0: about one second)
        self.buf = SymmetricBuffer(256, group)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.buf.device)   # barriers passed, kept on the device
        self.status = torch.zeros(1, dtype=torch.int32, device=self.buf.device)
        self.flag_table = self.buf.peer_table(0)
        if self.buf.world > 1:
            dist.barrier(group)          # every rank has mapped every flag array before the first signal

    def __call__(self) -> None:
        if self.buf.world == 1:
            return
        native.check(native.lib().lmb_peer_barrier(self.buf.local_ptr, self.flag_table.data_ptr(), self.buf.rank,
                                                   self.buf.world, self.epoch.data_ptr(), self.status.data_ptr(),
                                                   self.limit_cycles, native.stream_ptr()), "peer_barrier")

    def check(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"peer barrier timed out waiting for rank {code - 100}")

    def close(self) -> None:
        self.buf.close()

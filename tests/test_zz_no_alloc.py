"""Allocation-free prefix sum (``lmb_exclusive_scan_u32_noalloc``).

Some users of the kernel library cannot call ``cudaMalloc`` where they need a scan: a serving loop
that must not take the driver's allocation lock, or a plug-in living inside an application that
owns the whole memory budget.  For them the library keeps the scan's temporary storage in a fixed
device array.  This test drives that entry point through its exported C symbol and checks it
against the ordinary entry point (which takes a caller-allocated workspace), twice in a row, because
the second call starts from the workspace contents the first one left behind.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

from landmarksystem_b200.ops import build

pytestmark = pytest.mark.gpu

ERR_TOO_LARGE = -1001
MAX_ELEMS = 16 * 1024 * 1024


def _load():
    lib = ctypes.CDLL(str(build.library_path()))
    lib.lmb_exclusive_scan_u32_noalloc.restype = ctypes.c_int
    lib.lmb_exclusive_scan_u32_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p]
    lib.lmb_exclusive_scan_u32.restype = ctypes.c_int
    lib.lmb_exclusive_scan_u32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                                           ctypes.c_void_p]
    lib.lmb_scan_scratch_bytes.restype = ctypes.c_longlong
    lib.lmb_scan_scratch_bytes.argtypes = [ctypes.c_longlong]
    return lib


def _existing(lib, x):
    out = torch.empty_like(x)
    ws = torch.empty(lib.lmb_scan_scratch_bytes(x.numel()), dtype=torch.uint8, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.lmb_exclusive_scan_u32(x.data_ptr(), out.data_ptr(), x.numel(), ws.data_ptr(), stream) == 0
    return out


def test_noalloc_scan_matches_existing_entry_point_twice():
    lib = _load()
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(7)
    # two calls in a row with different sizes: the second one sees the first one's leftovers
    for n in (5_000_000, 123_457):
        x = torch.randint(0, 1000, (n,), dtype=torch.int32, device="cuda", generator=gen)
        got = torch.empty_like(x)
        rc = lib.lmb_exclusive_scan_u32_noalloc(x.data_ptr(), got.data_ptr(), n, stream)
        assert rc == 0, f"entry point returned {rc}"
        want = _existing(lib, x)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert torch.equal(got.long() & 0xFFFFFFFF, (torch.cumsum(x.long(), 0) - x.long()) & 0xFFFFFFFF)


def test_noalloc_scan_refuses_oversized_requests():
    lib = _load()
    x = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = lib.lmb_exclusive_scan_u32_noalloc(x.data_ptr(), x.data_ptr(), MAX_ELEMS + 1,
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == ERR_TOO_LARGE


def test_noalloc_scan_in_place_and_at_the_size_limit():
    """Two promises of the header: the output may be the input buffer, and exactly the maximum length is accepted."""
    lib = _load()
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(11)
    for n in (1_000_003, MAX_ELEMS):
        x = torch.randint(0, 200, (n,), dtype=torch.int32, device="cuda", generator=gen)
        want = _existing(lib, x)
        buf = x.clone()
        rc = lib.lmb_exclusive_scan_u32_noalloc(buf.data_ptr(), buf.data_ptr(), n, stream)
        assert rc == 0, f"entry point returned {rc}"
        torch.cuda.synchronize()
        assert torch.equal(buf, want)

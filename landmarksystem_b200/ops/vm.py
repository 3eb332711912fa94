"""VM feature-grid lookup op: CUDA kernel on GPU tensors, PyTorch math on CPU tensors.

Layout contract (channels-last): ``planes[l]`` is ``[B, H_l, W_l, C]``, ``lines[l]`` is
``[B, Z_l, C]``; ``coords`` is ``[N, 4]`` fp32 = block-local ``(x, y, z)`` in ``[-1, 1]`` plus the
block index (negative = sample is outside every block → zero features, zero gradient).
Output is ``[N, L*C]`` with level-major channel order, i.e. the concat-over-levels of
``plane ⊙ line`` that the reference builds from two ``F.grid_sample`` calls per level
(landmark/nerf_components/model_components/fields/encodings/tensor_vm_encoding.py:129-197).
"""
from __future__ import annotations

from ctypes import POINTER, byref, c_float, c_int, c_longlong
from typing import List, Optional, Sequence

import torch

from . import native


def _taps(u: torch.Tensor, size: int):
    f = (u + 1.0) * 0.5 * (size - 1)
    i0 = torch.floor(f)
    t = f - i0
    i0 = i0.long()
    i1 = i0 + 1
    w0 = torch.where((i0 >= 0) & (i0 < size), 1.0 - t, torch.zeros_like(t))
    w1 = torch.where((i1 >= 0) & (i1 < size), t, torch.zeros_like(t))
    return i0.clamp(0, size - 1), i1.clamp(0, size - 1), w0, w1


def vm_encode_reference(coords: torch.Tensor, planes: Sequence[torch.Tensor], lines: Sequence[torch.Tensor]) -> torch.Tensor:
    """Differentiable plain-PyTorch statement of the op (fp32 math); the numerics oracle."""
    x, y, z, bf = coords.unbind(-1)
    n_blocks = planes[0].shape[0]
    b = bf.long()
    ok = (b >= 0) & (b < n_blocks)
    bc = b.clamp(0, n_blocks - 1)
    feats = []
    for plane, line in zip(planes, lines):
        _, H, W, C = plane.shape
        Z = line.shape[1]
        x0, x1, wx0, wx1 = _taps(x, W)
        y0, y1, wy0, wy1 = _taps(y, H)
        z0, z1, wz0, wz1 = _taps(z, Z)
        pf = plane.float()
        lf = line.float()
        pv = (pf[bc, y0, x0] * (wy0 * wx0)[:, None] + pf[bc, y0, x1] * (wy0 * wx1)[:, None]
              + pf[bc, y1, x0] * (wy1 * wx0)[:, None] + pf[bc, y1, x1] * (wy1 * wx1)[:, None])
        lv = lf[bc, z0] * wz0[:, None] + lf[bc, z1] * wz1[:, None]
        feats.append(pv * lv * ok[:, None].to(pv.dtype))
    return torch.cat(feats, dim=-1)


def _levels_struct(planes, lines, gplanes=None, glines=None) -> native.VMLevels:
    lv = native.VMLevels()
    lv.L = len(planes)
    lv.B, _, _, lv.C = planes[0].shape
    for i, (p, l) in enumerate(zip(planes, lines)):
        assert p.is_contiguous() and l.is_contiguous(), "VM grids must be contiguous channels-last tensors"
        lv.plane[i] = p.data_ptr()
        lv.line[i] = l.data_ptr()
        lv.H[i], lv.W[i], lv.Z[i] = p.shape[1], p.shape[2], l.shape[1]
        if gplanes is not None:
            lv.gplane[i] = gplanes[i].data_ptr()
            lv.gline[i] = glines[i].data_ptr()
    return lv


# Backward flavour of the lookup: False = 16-byte vector reductions into the fp32 accumulators (fast, summation order
# varies from run to run); True = atomic-free sorted segmented sums (bit-reproducible, about 3x slower).
DETERMINISTIC_BACKWARD = False

native.register_signature("lmb_vm_encode_bwd_sorted", [native.P, native.P, c_longlong, POINTER(native.VMLevels), c_int, native.P,
                                                        c_int, c_int, native.P, native.P, native.P, native.P, native.P, native.P])
native.register_signature("lmb_radix_sort_scratch_bytes", [c_longlong])


def _sorted_backward(coords, count, lv, param_dtype, dout):
    n = coords.shape[0]
    dev = coords.device
    lib = native.lib()
    lib.lmb_radix_sort_scratch_bytes.restype = c_longlong
    scratch = torch.empty(int(lib.lmb_radix_sort_scratch_bytes(n)), dtype=torch.uint8, device=dev)
    pkeys = torch.empty(n, dtype=torch.int64, device=dev)
    zkeys = torch.empty(n, dtype=torch.int64, device=dev)
    pvals = torch.empty(n, dtype=torch.int32, device=dev)
    zvals = torch.empty(n, dtype=torch.int32, device=dev)
    native.check(lib.lmb_vm_encode_bwd_sorted(coords.data_ptr(), native.ptr(count), n, byref(lv), native.DTYPE_CODE[param_dtype],
                                              dout.data_ptr(), native.DTYPE_CODE[dout.dtype], dout.shape[1], pkeys.data_ptr(),
                                              pvals.data_ptr(), zkeys.data_ptr(), zvals.data_ptr(), scratch.data_ptr(),
                                              native.stream_ptr()), "vm_encode_bwd_sorted")


class _VMEncode(torch.autograd.Function):
    """Inputs: coords, count (or None), out_dtype, n_levels, shadow flag, then 2*L master tensors
    (planes..., lines...) and optionally 2*L bf16 shadow tensors that the kernels read instead."""

    @staticmethod
    def forward(ctx, coords, count, out_dtype, n_levels, out_width, zero_fill, tail, *grids):
        masters = grids[: 2 * n_levels]
        shadows = grids[2 * n_levels:]
        read = shadows if shadows else masters
        planes, lines = list(read[:n_levels]), list(read[n_levels:])
        N = coords.shape[0]
        C = planes[0].shape[-1]
        width = max(out_width, n_levels * C)
        out = torch.empty((N, width), device=coords.device, dtype=out_dtype)
        if zero_fill and (count is not None or width > n_levels * C):
            out.zero_()
        lv = _levels_struct(planes, lines)
        t_dirs, t_idx, t_spr, t_col = tail if tail is not None else (None, None, 1, 0)
        native.check(
            native.lib().lmb_vm_encode_fwd(coords.data_ptr(), native.ptr(count), N, byref(lv),
                                           native.DTYPE_CODE[planes[0].dtype], out.data_ptr(),
                                           native.DTYPE_CODE[out_dtype], width, native.ptr(t_dirs), native.ptr(t_idx),
                                           int(t_spr), int(t_col), native.stream_ptr()),
            "vm_encode_fwd")
        ctx.save_for_backward(coords, count, *read)
        ctx.n_levels = n_levels
        ctx.masters = masters
        ctx.n_shadow = len(shadows)
        return out

    @staticmethod
    def backward(ctx, dout):
        coords, count, *read = ctx.saved_tensors
        L = ctx.n_levels
        planes, lines = read[:L], read[L:]
        masters = ctx.masters
        grads = []
        sunk = []
        for m in masters:
            # A fused optimiser may attach a persistent, pre-zeroed fp32 accumulator (`_lmb_grad_sink`)
            # to a parameter; the kernel then adds into it directly and autograd gets no tensor, which
            # saves allocating and re-reading a multi-GB dense gradient every step.
            sink = getattr(m, "_lmb_grad_sink", None)
            sunk.append(sink is not None)
            grads.append(sink if sink is not None else torch.zeros(m.shape, device=m.device, dtype=torch.float32))
        lv = _levels_struct(planes, lines, grads[:L], grads[L:])
        dout = dout.contiguous()
        if DETERMINISTIC_BACKWARD:
            _sorted_backward(coords, count, lv, planes[0].dtype, dout)
        else:
            native.check(
                native.lib().lmb_vm_encode_bwd(coords.data_ptr(), native.ptr(count), coords.shape[0], byref(lv),
                                               native.DTYPE_CODE[planes[0].dtype], dout.data_ptr(),
                                               native.DTYPE_CODE[dout.dtype], dout.shape[1], native.stream_ptr()),
                "vm_encode_bwd")
        out_grads = [None if s else g for s, g in zip(sunk, grads)]
        return (None, None, None, None, None, None, None, *out_grads, *([None] * ctx.n_shadow))


def vm_encode(coords: torch.Tensor, planes: List[torch.Tensor], lines: List[torch.Tensor],
              shadow_planes: Optional[List[torch.Tensor]] = None, shadow_lines: Optional[List[torch.Tensor]] = None,
              count: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float32,
              out_width: int = 0, zero_fill: bool = True, tail=None) -> torch.Tensor:
    """Look up ``[N, L*C]`` features.  ``shadow_*`` (bf16 copies of the fp32 masters) are what the
    CUDA kernels read when given; gradients always flow to the fp32 masters.  ``out_width`` > L*C
    returns a wider, zero-padded row (room for columns a consumer kernel wants appended).  With
    ``zero_fill=False`` padding columns and rows past ``count`` are left uninitialised (for consumers
    that never read them).  ``tail = (dirs [R, 3] fp32, idx int32 [N] or None, samples_per_ray, col)``: the kernel also
    writes ``dirs[idx // samples_per_ray]`` (``dirs[row]`` without ``idx``) and 13 zeros into columns ``col .. col+15``."""
    if not coords.is_cuda:
        feat = vm_encode_reference(coords, planes, lines).to(out_dtype)
        if out_width > feat.shape[1]:
            feat = torch.nn.functional.pad(feat, (0, out_width - feat.shape[1]))
        if tail is not None:
            t_dirs, t_idx, t_spr, t_col = tail
            rows = t_dirs if t_idx is None else t_dirs[(t_idx.long() // t_spr)]
            feat[:, t_col:t_col + 16] = 0
            feat[: rows.shape[0], t_col:t_col + 3] = rows[: feat.shape[0]].to(out_dtype)
        return feat
    coords = coords.contiguous().float()
    grids = list(planes) + list(lines)
    if shadow_planes is not None:
        grids += list(shadow_planes) + list(shadow_lines)
    return _VMEncode.apply(coords, count, out_dtype, len(planes), out_width, zero_fill, tail, *grids)


# -- fused density head: lookup + 1-wide linear (or channel sum) + activation -> sigma [N] ---------------------
native.register_signature("lmb_vm_density_fwd", [native.P, native.P, c_longlong, POINTER(native.VMLevels), c_int, native.P,
                                                  c_int, c_int, c_float, native.P, native.P, native.P, native.P, native.P, c_int,
                                                  native.P])
native.register_signature("lmb_vm_density_bwd", [native.P, native.P, c_longlong, POINTER(native.VMLevels), c_int, native.P,
                                                  c_int, c_int, c_float, native.P, native.P, native.P, native.P])


def vm_density_supported(planes) -> bool:
    ch = planes[0].shape[-1] // 8
    return planes[0].is_cuda and planes[0].shape[-1] % 8 == 0 and 1 <= ch <= 32 and (ch & (ch - 1)) == 0


def vm_density_reference(coords, planes, lines, weight, inner_relu: bool, act: str, shift: float) -> torch.Tensor:
    feat = vm_encode_reference(coords, planes, lines)
    z = feat @ weight.reshape(-1).float() if weight is not None else feat.sum(-1)
    r = torch.relu(z) if inner_relu else z
    return torch.relu(r) if act == "relu" else torch.nn.functional.softplus(r + shift)


class _VMDensity(torch.autograd.Function):
    """Inputs: coords, count, weight (or None), inner_relu, act code, shift, n_levels, then the grids as in
    ``_VMEncode``.  Output: sigma ``[N]`` fp32 (rows past ``count`` undefined)."""

    @staticmethod
    def forward(ctx, coords, count, weight, inner_relu, act, shift, n_levels, route, *grids):
        masters = grids[: 2 * n_levels]
        shadows = grids[2 * n_levels:]
        read = shadows if shadows else masters
        planes, lines = list(read[:n_levels]), list(read[n_levels:])
        N = coords.shape[0]
        sigma = torch.empty(N, device=coords.device, dtype=torch.float32)
        pre = torch.empty(N, device=coords.device, dtype=torch.float32)
        w = None if weight is None else weight.detach().reshape(-1).float().contiguous()
        lv = _levels_struct(planes, lines)
        # route = (src int32 [N], slot int32 [N], table of landing-buffer addresses, world): sigma also goes to its source rank
        r_src, r_slot, r_table, r_world = route if route is not None else (None, None, None, 0)
        native.check(native.lib().lmb_vm_density_fwd(coords.data_ptr(), native.ptr(count), N, byref(lv),
                                                     native.DTYPE_CODE[planes[0].dtype], native.ptr(w), int(inner_relu), act,
                                                     float(shift), sigma.data_ptr(), pre.data_ptr(), native.ptr(r_src),
                                                     native.ptr(r_slot), r_table, int(r_world), native.stream_ptr()),
                     "vm_density_fwd")
        ctx.save_for_backward(coords, count, pre, w, *read)
        ctx.n_levels, ctx.masters, ctx.n_shadow = n_levels, masters, len(shadows)
        ctx.head = (int(inner_relu), act, float(shift))
        ctx.weight_shape = None if weight is None else weight.shape
        return sigma

    @staticmethod
    def backward(ctx, dsigma):
        coords, count, pre, w, *read = ctx.saved_tensors
        L = ctx.n_levels
        planes, lines = read[:L], read[L:]
        grads, sunk = [], []
        for m in ctx.masters:
            sink = getattr(m, "_lmb_grad_sink", None)
            sunk.append(sink is not None)
            grads.append(sink if sink is not None else torch.zeros(m.shape, device=m.device, dtype=torch.float32))
        lv = _levels_struct(planes, lines, grads[:L], grads[L:])
        dw = None if w is None else torch.zeros_like(w)
        dsigma = dsigma.contiguous().float()
        native.check(native.lib().lmb_vm_density_bwd(coords.data_ptr(), native.ptr(count), coords.shape[0], byref(lv),
                                                     native.DTYPE_CODE[planes[0].dtype], native.ptr(w), *ctx.head,
                                                     dsigma.data_ptr(), pre.data_ptr(), native.ptr(dw), native.stream_ptr()),
                     "vm_density_bwd")
        out_grads = [None if s else g for s, g in zip(sunk, grads)]
        dweight = None if dw is None else dw.view(ctx.weight_shape)
        return (None, None, dweight, None, None, None, None, None, *out_grads, *([None] * ctx.n_shadow))


def vm_density(coords: torch.Tensor, planes, lines, shadow_planes=None, shadow_lines=None, weight=None,
               inner_relu: bool = False, act: str = "softplus", shift: float = 0.0, count=None, route=None) -> torch.Tensor:
    """``sigma [N] = act(relu?(features @ weight))`` (``weight=None``: plain channel sum) without materialising
    the features.  ``act``: ``"relu"`` or ``"softplus"`` (of ``x + shift``).  ``route`` (CUDA only): ``(src, slot, table,
    world)`` - the kernel also stores row ``n``'s density at ``slot[n]`` of rank ``src[n]``'s landing buffer (peer store)."""
    if not coords.is_cuda:
        return vm_density_reference(coords, planes, lines, weight, inner_relu, act, shift)
    coords = coords.contiguous().float()
    grids = list(planes) + list(lines)
    if shadow_planes is not None:
        grids += list(shadow_planes) + list(shadow_lines)
    return _VMDensity.apply(coords, count, weight, inner_relu, 0 if act == "relu" else 1, shift, len(planes), route, *grids)

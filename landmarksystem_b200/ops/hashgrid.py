"""Multiresolution hash-grid encoding (Instant-NGP style), forward and backward.

Geometry follows the public tiny-cuda-nn definition the reference relies on through
``tcnn.Encoding("HashGrid")`` (landmark/nerf_components/model_components/fields/encodings/
hash_encoding.py:82-107): level ``l`` has ``scale_l = base * growth^l - 1``, resolution
``ceil(scale_l) + 1``, sample position ``x * scale_l + 0.5``; a level whose dense grid fits its
table is indexed densely, otherwise by the XOR-of-primes spatial hash; trilinear interpolation of
``F`` features per entry.  Tables of all levels are concatenated into one parameter
``[sum(entries_l), F]``.

CPU tensors run the PyTorch statement below (the oracle); CUDA tensors run ``csrc/hashgrid.cu``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List

import torch

from . import native

_PRIMES = (1, 2654435761, 805459861)


@dataclass
class HashGridMeta:
    n_levels: int
    n_features: int
    log2_hashmap_size: int
    base_resolution: int
    per_level_scale: float
    scales: List[float]
    resolutions: List[int]
    offsets: List[int]      # entry offset of each level (len n_levels + 1)

    @property
    def n_params(self) -> int:
        return self.offsets[-1] * self.n_features

    @property
    def out_dim(self) -> int:
        return self.n_levels * self.n_features


def make_meta(n_levels: int, n_features: int, log2_hashmap_size: int, base_resolution: int,
              per_level_scale: float) -> HashGridMeta:
    scales, resolutions, offsets = [], [], [0]
    cap = 1 << log2_hashmap_size
    for l in range(n_levels):
        scale = math.exp2(l * math.log2(per_level_scale)) * base_resolution - 1.0
        res = int(math.ceil(scale)) + 1
        entries = min(((res ** 3 + 7) // 8) * 8, cap) if res ** 3 < (1 << 62) else cap
        scales.append(scale)
        resolutions.append(res)
        offsets.append(offsets[-1] + entries)
    return HashGridMeta(n_levels, n_features, log2_hashmap_size, base_resolution, per_level_scale, scales,
                        resolutions, offsets)


def _index(ix, iy, iz, res: int, entries: int):
    if res ** 3 <= entries:
        return ix + iy * res + iz * res * res
    h = (ix * _PRIMES[0]) ^ (iy * _PRIMES[1]) ^ (iz * _PRIMES[2])
    return (h & 0xFFFFFFFF) % entries


def hashgrid_reference(x: torch.Tensor, table: torch.Tensor, meta: HashGridMeta) -> torch.Tensor:
    """``x [N, 3]`` in ``[0, 1]``, ``table [entries, F]`` -> ``[N, L*F]`` (differentiable w.r.t. table)."""
    outs = []
    tab = table.float()
    for l in range(meta.n_levels):
        scale, res = meta.scales[l], meta.resolutions[l]
        off, entries = meta.offsets[l], meta.offsets[l + 1] - meta.offsets[l]
        pos = x.float() * scale + 0.5
        p0 = torch.floor(pos)
        w = pos - p0
        p0 = p0.long()
        acc = 0
        for dz in (0, 1):
            for dy in (0, 1):
                for dx in (0, 1):
                    ix = (p0[:, 0] + dx).clamp(0, res - 1)
                    iy = (p0[:, 1] + dy).clamp(0, res - 1)
                    iz = (p0[:, 2] + dz).clamp(0, res - 1)
                    wt = ((w[:, 0] if dx else 1 - w[:, 0]) * (w[:, 1] if dy else 1 - w[:, 1])
                          * (w[:, 2] if dz else 1 - w[:, 2]))
                    acc = acc + tab[off + _index(ix, iy, iz, res, entries)] * wt[:, None]
        outs.append(acc)
    return torch.cat(outs, dim=-1)


class _LevelMeta(native.Structure):
    _fields_ = [("scale", native.c_float * 32), ("res", native.c_int * 32), ("offset", native.c_longlong * 33),
                ("n_levels", native.c_int), ("n_features", native.c_int)]


def _meta_struct(meta: HashGridMeta) -> "_LevelMeta":
    s = _LevelMeta()
    assert meta.n_levels <= 32
    for l in range(meta.n_levels):
        s.scale[l], s.res[l], s.offset[l] = meta.scales[l], meta.resolutions[l], meta.offsets[l]
    s.offset[meta.n_levels] = meta.offsets[-1]
    s.n_levels, s.n_features = meta.n_levels, meta.n_features
    return s


native.register_signature("lmb_hashgrid_fwd", [native.P, native.c_longlong, native.P, native.c_int,
                                                native.POINTER(_LevelMeta), native.P, native.c_int, native.P])
native.register_signature("lmb_hashgrid_bwd", [native.P, native.c_longlong, native.POINTER(_LevelMeta), native.P,
                                                native.c_int, native.P, native.P])


class _HashGrid(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, table, meta, out_dtype, shadow, sink, precomputed):
        read = shadow if shadow is not None else table
        if precomputed is not None:
            # the caller already looked these samples up with the same table (the sampler's density query of this
            # step): only the backward runs here
            assert precomputed.shape == (x.shape[0], meta.out_dim)
            out = precomputed.view_as(precomputed)
        else:
            out = torch.empty((x.shape[0], meta.out_dim), device=x.device, dtype=out_dtype)
            ms = _meta_struct(meta)
            native.check(native.lib().lmb_hashgrid_fwd(x.data_ptr(), x.shape[0], read.data_ptr(),
                                                       native.DTYPE_CODE[read.dtype], ctx_ref(ms), out.data_ptr(),
                                                       native.DTYPE_CODE[out_dtype], native.stream_ptr()), "hashgrid_fwd")
        ctx.save_for_backward(x)
        ctx.meta, ctx.table, ctx.sink = meta, table, sink
        return out

    @staticmethod
    def backward(ctx, dout):
        (x,) = ctx.saved_tensors
        table, meta = ctx.table, ctx.meta
        sink = ctx.sink if ctx.sink is not None else getattr(table, "_lmb_grad_sink", None)
        grad = sink if sink is not None else torch.zeros(table.shape, device=table.device, dtype=torch.float32)
        dout = dout.contiguous()
        ms = _meta_struct(meta)
        native.check(native.lib().lmb_hashgrid_bwd(x.data_ptr(), x.shape[0], ctx_ref(ms), dout.data_ptr(),
                                                   native.DTYPE_CODE[dout.dtype], grad.data_ptr(),
                                                   native.stream_ptr()), "hashgrid_bwd")
        return None, (None if sink is not None else grad), None, None, None, None, None


def ctx_ref(struct):
    from ctypes import byref

    return byref(struct)


def hashgrid_encode(x: torch.Tensor, table: torch.Tensor, meta: HashGridMeta, out_dtype: torch.dtype = torch.float32,
                    shadow: torch.Tensor = None, sink: torch.Tensor = None, precomputed: torch.Tensor = None) -> torch.Tensor:
    """``shadow``: bf16 copy of ``table`` for the kernel to read; ``sink``: persistent fp32 accumulator that receives the
    table gradient instead of a fresh tensor (both default to the attributes a fused optimiser attached to ``table``);
    ``precomputed``: the result of an earlier lookup of the same samples with the same table - returned as is, so that only
    the backward is computed."""
    if table.numel() < meta.n_params:           # a table smaller than the level layout would be read out of bounds
        raise ValueError(f"hash table holds {table.numel()} values, the level layout needs {meta.n_params}")
    if not x.is_cuda:
        return hashgrid_reference(x, table, meta).to(out_dtype)
    if shadow is None:
        shadow = getattr(table, "_lmb_shadow", None)
    return _HashGrid.apply(x.contiguous().float(), table, meta, out_dtype, shadow, sink, precomputed)

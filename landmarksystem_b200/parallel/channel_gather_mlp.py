"""Channel-parallel colour head with the all-gather fused into the first GEMM.

With feature channels split across P ranks, every rank looks all samples up on its ``C/P`` channel
slice.  The reference then all-gathers plane and line features (NCCL list all-gather + host sync,
landmark/nerf_components/model_components/fields/encodings/tensor_vm_encoding.py:421-435) before the
decoder.  Here each rank writes its ``plane * line`` slice into a symmetric buffer and the tcgen05
colour-head kernel builds its input tile from P column ranges: the local range comes from local HBM,
every other range is pulled from the peer's buffer over NVLink by the kernel's own (non-multicast)
TMA loads, tile by tile, overlapping with the tensor-core work of other tiles.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_longlong, c_void_p
from typing import List

import torch

from ..comm.symmetric import PeerBarrier, SymmetricBuffer
from ..ops import fused_mlp, native

native.register_signature("lmb_fused_mlp_fwd_multi", [native.P, native.P, c_int, native.P, c_longlong, native.P,
                                                       ctypes.POINTER(fused_mlp.MLPSpec), native.P, c_int, native.P,
                                                       native.P])


class ChannelGatherColourHead:
    """Runs ``RGBDecoder`` for ``max_rows`` samples whose features are channel-sliced over ``group``."""

    def __init__(self, decoder, n_levels: int, channels_per_rank: int, max_rows: int, group=None):
        self.decoder, self.L, self.cl = decoder, n_levels, channels_per_rank
        self.width = n_levels * channels_per_rank
        assert self.width % 8 == 0, "per-rank feature width must be a multiple of 8"
        self.max_rows = max_rows
        self.buf = SymmetricBuffer(max_rows * self.width * 2, group)
        self.rank, self.world = self.buf.rank, self.buf.world
        assert self.world * self.width <= 144 and self.world + 1 <= 4, "fused colour head supports <= 3 channel slices"
        self.feat = self.buf.view(0, (max_rows, self.width), torch.bfloat16)
        self.dirs = torch.zeros(max_rows, 16, dtype=torch.bfloat16, device=self.buf.device)
        self.barrier = PeerBarrier(group)
        self.packed = None

    def _packed(self) -> fused_mlp.PackedMLP:
        dec = self.decoder
        if self.packed is None or self.packed.layers[1][0] is not dec.decoder.linears()[0].weight:
            lin = dec.decoder.linears()
            P, L, cl = self.world, self.L, self.cl
            C = P * cl
            # input columns arrive as [rank][level][channel]; the checkpoint's basis expects [level][rank][channel]
            perm = torch.tensor([l * C + p * cl + c for p in range(P) for l in range(L) for c in range(cl)],
                                device=dec.basis_mat.weight.device)
            self._perm = perm
            self._basis_view = dec.basis_mat.weight      # keep identity for cache validation
            layers = [(dec.basis_mat.weight, None, "none"), (lin[0].weight, lin[0].bias, "relu"),
                      (lin[1].weight, lin[1].bias, "relu"), (lin[2].weight, lin[2].bias, "sigmoid")]
            packed = fused_mlp.PackedMLP(layers, in_width=P * self.width + 16, out_dim=3, pe_stage=True,
                                         dir_col=P * self.width, k_override=[fused_mlp._pad16(P * self.width), 160, 128, 128])
            original_refresh = packed.refresh

            def refresh():
                # pack with the permuted basis columns - only when a weight changed since the last packing
                w = dec.basis_mat.weight
                if packed.blob is not None and packed.versions == packed._versions():
                    return
                permuted = w.detach()[:, perm]
                packed.layers = [(permuted, None, "none")] + packed.layers[1:]
                packed.versions = None
                original_refresh()
                packed.layers = [(w, None, "none")] + packed.layers[1:]
                packed.versions = packed._versions()          # versions of the real parameters, not of the permuted copy

            packed.refresh_permuted = refresh
            self.packed = packed
        return self.packed

    @torch.no_grad()
    def __call__(self, local_features: torch.Tensor, dirs: torch.Tensor) -> torch.Tensor:
        """``local_features [N, L * C/P]`` (this rank's channel slice, level-major), ``dirs [N, 3]`` -> rgb ``[N, 3]``."""
        N = local_features.shape[0]
        assert N <= self.max_rows
        packed = self._packed()
        packed.refresh_permuted()
        self.feat[:N].copy_(local_features)
        self.dirs[:N, :3].copy_(dirs)
        self.barrier()                               # every rank's slice is in its buffer
        ptrs = [self.buf.peer_ptrs[p] for p in range(self.world)] + [self.dirs.data_ptr()]
        widths = [self.width] * self.world + [16]
        xs = (c_void_p * len(ptrs))(*ptrs)
        ws = (c_int * len(widths))(*widths)
        out = torch.empty(N, 3, device=local_features.device, dtype=torch.float32)
        native.check(native.lib().lmb_fused_mlp_fwd_multi(xs, ws, len(ptrs), None, N, packed.blob.data_ptr(),
                                                          byref(packed.spec), out.data_ptr(), 3,
                                                          packed.status.data_ptr(), native.stream_ptr()),
                     "fused_mlp_fwd_multi")
        self.barrier()                               # peers have finished reading before anyone overwrites
        return out

"""Python side of the tcgen05 fused-MLP kernel (``csrc/fused_mlp.cu``).

Weights of a whole network are packed once (and re-packed when their version counters change) into
one device blob in the shared-memory operand layout ``[K/8][N][8]`` bf16 + fp32 biases, which the
kernel pulls in with a single TMA bulk copy.  Supported: up to 5 layers, every padded layer width
<= 160, activations none/relu/sigmoid/tanh/exp.  ``rgb_decoder_*`` drives the GridNeRF colour head
(basis projection + sin/cos expansion + 3-layer decoder) as one kernel.

Training backward runs in one tcgen05 kernel (``csrc/fused_mlp_bwd.cu``: recompute, data gradients and weight
gradients in one launch) for the GridNeRF colour head and for plain two- / three-layer relu networks up to
159 -> 128 -> 128 -> 16 (the 64-wide heads of the hash-grid models); other networks recompute with PyTorch
ops under bf16 autocast.
"""
from __future__ import annotations

from ctypes import POINTER, Structure, byref, c_int, c_longlong
from typing import List, Optional, Sequence, Tuple

import torch

from . import native

MAX_LAYERS, MAX_K, MAX_N = 5, 160, 160
MLP3_BACKWARD_KERNEL = True      # plain 2/3-layer networks: backward through the tcgen05 kernel instead of PyTorch ops
ACT = {"none": 0, "relu": 1, "sigmoid": 2, "tanh": 3, "exp": 4}


class MLPSpec(Structure):
    _fields_ = [("n_layers", c_int), ("K", c_int * MAX_LAYERS), ("N", c_int * MAX_LAYERS), ("act", c_int * MAX_LAYERS),
                ("w_off", c_int * MAX_LAYERS), ("b_off", c_int * MAX_LAYERS), ("blob_bytes", c_int),
                ("in_width", c_int), ("out_dim", c_int), ("pe_stage", c_int), ("dir_col", c_int), ("bias_in_gemm", c_int), ("hidden_cols", c_int)]


native.register_signature("lmb_fused_mlp_fwd", [native.P, native.P, c_longlong, native.P, POINTER(MLPSpec), native.P,
                                                 c_int, native.P, native.P])
native.register_signature("lmb_rgb_mlp_bwd", [native.P, native.P, c_longlong, native.P, POINTER(MLPSpec), native.P, c_int,
                                               native.P, native.P, native.P, native.P])
native.register_signature("lmb_rgb_mlp_bwd_gbuf_floats", [])
native.register_signature("lmb_mlp3_bwd", [native.P, c_int, native.P, c_longlong, native.P, POINTER(MLPSpec), native.P, c_int,
                                            native.P, native.P, native.P, native.P])


def _pad16(v: int) -> int:
    return (v + 15) // 16 * 16


def _act_name(module) -> str:
    if module is None:
        return "none"
    name = type(module).__name__.lower()
    return {"relu": "relu", "sigmoid": "sigmoid", "tanh": "tanh"}.get(name, "unsupported")


def pack_weight(w: torch.Tensor, n_pad: int, k_pad: int, bias: Optional[torch.Tensor] = None,
                bias_col: Optional[int] = None) -> torch.Tensor:
    """``[N, K]`` -> bf16 ``[k_pad/8, n_pad, 8]`` flattened (zero padded); ``bias`` goes into column ``bias_col``."""
    full = torch.zeros(n_pad, k_pad, device=w.device, dtype=torch.float32)
    full[: w.shape[0], : w.shape[1]] = w.detach().float()
    if bias is not None:
        full[: bias.shape[0], bias_col] = bias.detach().float()
    return full.view(n_pad, k_pad // 8, 8).permute(1, 0, 2).contiguous().to(torch.bfloat16).view(-1)


class PackedMLP:
    """Device blob + spec for a list of ``(weight [N,K], bias or None, activation)`` layers."""

    def __init__(self, layers: Sequence[Tuple[torch.Tensor, Optional[torch.Tensor], str]], in_width: int,
                 out_dim: int, pe_stage: bool = False, dir_col: int = 0, k_override: Optional[List[int]] = None,
                 bias_cols: Optional[dict] = None):
        """``bias_cols``: ``{layer: column}`` - the layer's bias is written into that (otherwise zero) column of its padded
        weights, which the kernels multiply with a ones column of the layer's input, so the epilogue adds nothing."""
        self.bias_cols = bias_cols or {}
        self.layers = layers
        self.in_width, self.out_dim, self.pe_stage, self.dir_col, self.k_override = in_width, out_dim, pe_stage, dir_col, k_override
        self.versions = None
        self.blob = None
        self.spec = None
        self.status = None

    def _versions(self):
        from . import optim

        return (optim.GENERATION,) + tuple((w._version, None if b is None else b._version) for w, b, _ in self.layers)

    def refresh(self):
        if self.versions == self._versions() and self.blob is not None:
            return
        dev = self.layers[0][0].device
        spec = MLPSpec()
        spec.n_layers = len(self.layers)
        parts, off = [], 0
        for l, (w, b, act) in enumerate(self.layers):
            k_pad = self.k_override[l] if self.k_override else _pad16(w.shape[1])
            n_pad = _pad16(w.shape[0])
            assert k_pad <= MAX_K and n_pad <= MAX_N, "layer too wide for the fused kernel"
            spec.K[l], spec.N[l], spec.act[l] = k_pad, n_pad, ACT[act]
            col = self.bias_cols.get(l) if b is not None else None
            if col is not None:
                assert w.shape[1] <= col < k_pad, "bias column must lie in the zero padding of the weights"
                spec.bias_in_gemm |= 1 << l
            packed = pack_weight(w, n_pad, k_pad, b if col is not None else None, col).view(torch.uint8)
            spec.w_off[l] = off
            parts.append(packed)
            off += packed.numel()
            if b is not None:
                bias = torch.zeros(n_pad, device=dev, dtype=torch.float32)
                bias[: b.shape[0]] = b.detach().float()
                spec.b_off[l] = off
                parts.append(bias.view(torch.uint8))
                off += n_pad * 4
            else:
                spec.b_off[l] = -1
        pad = (-off) % 16
        if pad:
            parts.append(torch.zeros(pad, device=dev, dtype=torch.uint8))
            off += pad
        spec.blob_bytes, spec.in_width, spec.out_dim = off, self.in_width, self.out_dim
        spec.pe_stage, spec.dir_col = int(self.pe_stage), self.dir_col
        self.blob = torch.cat(parts).contiguous()
        self.spec = spec
        self.versions = self._versions()
        if self.status is None:
            self.status = torch.zeros(1, device=dev, dtype=torch.int32)

    def run(self, x: torch.Tensor, count: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x [N, in_width]`` bf16 contiguous -> fp32 ``[N, out_dim]``."""
        self.refresh()
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == self.in_width
        out = torch.empty((x.shape[0], self.out_dim), device=x.device, dtype=torch.float32)
        if count is not None:
            out.zero_()
        native.check(native.lib().lmb_fused_mlp_fwd(x.data_ptr(), native.ptr(count), x.shape[0], self.blob.data_ptr(),
                                                    byref(self.spec), out.data_ptr(), self.out_dim,
                                                    self.status.data_ptr(), native.stream_ptr()), "fused_mlp_fwd")
        return out

    def check_status(self) -> None:
        """Host-side read of the kernel's error word (a bounded wait that expired); call off the hot path."""
        code = int(self.status.item()) if self.status is not None else 0
        if code:
            raise RuntimeError(f"fused MLP kernel reported status {code} (1: weights, 2: input tile, 3: MMA wait)")


# -- generic MLPDecoder -----------------------------------------------------------------------
def _decoder_layers(decoder):
    linears = decoder.linears()
    out_act = _act_name(decoder.out_activation)
    layers = []
    for i, lin in enumerate(linears):
        act = "relu" if i < len(linears) - 1 else out_act
        layers.append((lin.weight, lin.bias, act))
    return layers


def fused_mlp_supported(decoder) -> bool:
    if not native.available():
        return False
    layers = _decoder_layers(decoder)
    if len(layers) > MAX_LAYERS or any(a == "unsupported" for _, _, a in layers):
        return False
    return all(_pad16(w.shape[0]) <= MAX_N and _pad16(w.shape[1]) <= MAX_K for w, _, _ in layers)


def _torch_mlp(x, layers, acts):
    h = x
    for (w, b), act in zip(layers, acts):
        h = torch.nn.functional.linear(h, w, b)
        if act == "relu":
            h = torch.relu(h)
        elif act == "sigmoid":
            h = torch.sigmoid(h)
        elif act == "tanh":
            h = torch.tanh(h)
        elif act == "exp":
            h = torch.exp(h)
    return h


# -- plain two- / three-layer networks: backward in one kernel -----------------------------------------------
MLP3_IN, MLP3_HID, MLP3_OUT, MLP3_ONES = 160, 128, 16, 159


def mlp3_backward_supported(packed: "PackedMLP") -> bool:
    """Two or three linear layers, relu between them, identity or sigmoid at the end, at most 159 inputs, 128 hidden
    units and 16 outputs."""
    layers = packed.layers
    if not native.available() or packed.pe_stage or len(layers) not in (2, 3):
        return False
    if any(a != "relu" for _, _, a in layers[:-1]) or layers[-1][2] not in ("none", "sigmoid"):
        return False
    return (layers[0][0].shape[1] <= MLP3_ONES and all(w.shape[0] <= MLP3_HID for w, _, _ in layers[:-1])
            and layers[-1][0].shape[0] <= MLP3_OUT)


class _PackedMLP3:
    """The network zero-padded to 160 -> 128 -> 128 -> 16 in the kernel's blob layout (a two-layer network keeps the
    blob's middle slot - an identity - but marks it so that the kernel skips that layer).  Re-packed when the optimiser generation or a parameter version moves."""

    def __init__(self, layers):
        self.layers, self.key, self.blob, self.spec, self.status = layers, None, None, None, None

    def refresh(self):
        from . import optim

        key = (optim.GENERATION,) + tuple((w._version, None if b is None else b._version) for w, b, _ in self.layers)
        if key == self.key:
            return
        dev = self.layers[0][0].device
        (w1, b1, _), (w3, b3, act3) = self.layers[0], self.layers[-1]
        if len(self.layers) == 3:
            w2, b2 = self.layers[1][0], self.layers[1][1]
        else:
            w2, b2 = torch.eye(MLP3_HID, device=dev), None
        spec = MLPSpec()
        spec.n_layers = 3
        parts, off = [], 0
        for l, (w, b, n_pad, k_pad, act) in enumerate(((w1, b1, MLP3_HID, MLP3_IN, "relu"), (w2, b2, MLP3_HID, MLP3_HID, "relu"),
                                                       (w3, b3, MLP3_OUT, MLP3_HID, act3))):
            spec.K[l], spec.N[l], spec.act[l] = k_pad, n_pad, ACT[act]
            packed = pack_weight(w, n_pad, k_pad).view(torch.uint8)
            spec.w_off[l] = off
            parts.append(packed)
            off += packed.numel()
            bias = torch.zeros(n_pad, device=dev, dtype=torch.float32)
            if b is not None:
                bias[: b.shape[0]] = b.detach().float()
            spec.b_off[l] = off
            parts.append(bias.view(torch.uint8))
            off += n_pad * 4
        spec.blob_bytes, spec.in_width, spec.out_dim, spec.pe_stage, spec.dir_col = off, MLP3_IN, w3.shape[0], 0, 0
        # layers without a bias (the hash-grid heads): the kernel skips the bias adds of its recompute epilogues
        spec.bias_in_gemm = (1 if b1 is None else 0) | (2 if b2 is None else 0)
        if len(self.layers) == 2:
            spec.K[1] = 0        # two-layer network: the kernel feeds h1 to the output layer and skips the middle layer
        spec.hidden_cols = max(w.shape[0] for w, _, _ in self.layers[:-1])      # <= 64: the kernel's epilogues walk 64 columns
        self.blob, self.spec, self.key = torch.cat(parts).contiguous(), spec, key
        if self.status is None:
            self.status = torch.zeros(1, device=dev, dtype=torch.int32)


def mlp3_backward(packed: "PackedMLP", x: torch.Tensor, dout: torch.Tensor):
    """``x [N, in_width]`` bf16 (the forward kernel's input), ``dout [N, out]`` -> (``dx`` bf16 ``[N, in_width]``, gradients
    in the order of the decoder's parameters: weight, bias (if any) per layer)."""
    p3 = getattr(packed, "_mlp3", None)
    if p3 is None:
        p3 = packed._mlp3 = _PackedMLP3(packed.layers)
    p3.refresh()
    if packed.status is not None:
        p3.status = packed.status          # one status word per network: ``PackedMLP.check_status`` covers both kernels
    lib = native.lib()
    n, k0 = x.shape[0], packed.layers[0][0].shape[1]
    gbuf = torch.zeros(int(lib.lmb_rgb_mlp_bwd_gbuf_floats()), device=x.device, dtype=torch.float32)
    dout = dout.contiguous().float()
    direct = x.shape[1] <= MLP3_IN - 8 and x.is_contiguous()
    if direct:
        # the kernel reads the rows as they are and supplies the zero and ones columns of its 160-wide operand itself:
        # no padded copy of the input, no padded gradient to slice
        xin, dx = x, torch.empty_like(x)
    else:
        xin = torch.zeros(n, MLP3_IN, device=x.device, dtype=torch.bfloat16)
        xin[:, :k0] = x[:, :k0]
        xin[:, MLP3_ONES] = 1.0
        dx = torch.empty_like(xin)
    native.check(lib.lmb_mlp3_bwd(xin.data_ptr(), xin.shape[1], None, n, p3.blob.data_ptr(), byref(p3.spec), dout.data_ptr(),
                                  dout.shape[1], dx.data_ptr(), gbuf.data_ptr(), p3.status.data_ptr(), native.stream_ptr()),
                 "mlp3_bwd")
    g1 = gbuf[: 128 * 160].view(128, 160)
    g2 = gbuf[128 * 160: 128 * 160 + 128 * 144].view(128, 144)
    o = 128 * 160 + 128 * 144
    g3t = gbuf[o: o + 128 * 16].view(128, 16)
    db3 = gbuf[o + 128 * 16 + 144 * 32: o + 128 * 16 + 144 * 32 + 16]
    layers = packed.layers
    n1, n_out = layers[0][0].shape[0], layers[-1][0].shape[0]
    grads = [g1[:n1, :k0].contiguous()]
    if layers[0][1] is not None:
        grads.append(g1[:n1, MLP3_ONES].contiguous())
    if len(layers) == 3:
        n2 = layers[1][0].shape[0]
        grads.append(g2[:n2, :n1].contiguous())
        if layers[1][1] is not None:
            grads.append(g2[:n2, 128].contiguous())
    else:
        n2 = n1
    grads.append(g3t[:n2, :n_out].t().contiguous())
    if layers[-1][1] is not None:
        grads.append(db3[:n_out].contiguous())
    if direct:
        return dx, grads
    dx_out = torch.zeros_like(x)
    dx_out[:, :k0] = dx[:, :k0]
    return dx_out, grads


class _FusedMLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, packed, n_params, precomputed, *params):
        ctx.packed, ctx.n_params = packed, n_params
        ctx.save_for_backward(x, *params)
        if precomputed is not None:           # the same rows went through the same weights earlier in this step
            return precomputed.view_as(precomputed)
        return packed.run(x)

    @staticmethod
    def backward(ctx, dout):
        x, *params = ctx.saved_tensors
        packed = ctx.packed
        if MLP3_BACKWARD_KERNEL and mlp3_backward_supported(packed):
            dx, grads = mlp3_backward(packed, x, dout)
            return (dx if ctx.needs_input_grad[0] else None, None, None, None, *grads)
        with torch.enable_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            xin = x.detach().requires_grad_(x.is_floating_point())
            leaves = [p.detach().requires_grad_() for p in params]
            pairs, it = [], iter(leaves)
            for w, b, _ in packed.layers:
                pairs.append((next(it), next(it) if b is not None else None))
            k0 = packed.layers[0][0].shape[1]
            out = _torch_mlp(xin[:, :k0], pairs, [a for _, _, a in packed.layers]).float()
            grads = torch.autograd.grad(out[:, : packed.out_dim], [xin] + leaves, dout, allow_unused=True)
        return (grads[0], None, None, None, *grads[1:])


class _CatPadBf16(torch.autograd.Function):
    """``[N, w_i]`` parts -> one bf16 ``[N, width]`` row block (zero tail): the concatenate, the padding and the cast of
    the kernel's input in one write pass; the backward hands each part its slice of the gradient."""

    @staticmethod
    def forward(ctx, width, *parts):
        n = parts[0].shape[0]
        out = torch.empty(n, width, device=parts[0].device, dtype=torch.bfloat16)
        col = 0
        for part in parts:
            out[:, col:col + part.shape[1]].copy_(part)
            col += part.shape[1]
        if col < width:
            out[:, col:].zero_()
        ctx.meta = [(part.shape[1], part.dtype) for part in parts]
        return out

    @staticmethod
    def backward(ctx, dout):
        grads, col = [], 0
        for k, (w, dtype) in enumerate(ctx.meta):
            grads.append(dout[:, col:col + w].to(dtype) if ctx.needs_input_grad[k + 1] else None)
            col += w
        return (None, *grads)


def mlp_forward(decoder, features, precomputed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``features``: ``[N, K]`` tensor or a sequence of ``[N, k_i]`` tensors that are concatenated along the last
    dimension while the kernel's bf16 input is written.  ``precomputed``: the network's fp32 output for exactly these
    rows, evaluated earlier with the same weights - no forward launch, the backward is recorded as usual."""
    packed = getattr(decoder, "_lmb_packed", None)
    layers = _decoder_layers(decoder)
    in_width = (layers[0][0].shape[1] + 7) // 8 * 8
    if packed is None or packed.layers[0][0] is not layers[0][0]:
        packed = PackedMLP(layers, in_width=_pad16(layers[0][0].shape[1]), out_dim=layers[-1][0].shape[0])
        decoder._lmb_packed = packed
    if isinstance(features, (tuple, list)):
        x = _CatPadBf16.apply(packed.in_width, *features)
    elif features.shape[1] != packed.in_width or features.dtype != torch.bfloat16:
        x = _CatPadBf16.apply(packed.in_width, features)
    else:
        x = features.contiguous()
    params = [t for w, b, _ in layers for t in ((w, b) if b is not None else (w,))]
    if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in params)):
        return _FusedMLPFn.apply(x, packed, len(params), precomputed, *params)
    return precomputed if precomputed is not None else packed.run(x)


# -- GridNeRF colour head ---------------------------------------------------------------------------
RGB_IN_WIDTH = 160


def rgb_decoder_supported(decoder) -> bool:
    if not native.available() or decoder.encode_app:
        return False
    lin = decoder.decoder.linears()
    return (decoder.app_dim == 27 and decoder.feape == 2 and decoder.viewpe == 2 and len(lin) == 3
            and decoder.basis_mat.weight.shape[1] <= 144 and lin[0].weight.shape == (lin[0].weight.shape[0], 150)
            and lin[0].weight.shape[0] <= 128 and isinstance(decoder.decoder.out_activation, torch.nn.Sigmoid))


def _rgb_packed(decoder) -> PackedMLP:
    packed = getattr(decoder, "_lmb_packed", None)
    if packed is None or packed.layers[0][0] is not decoder.basis_mat.weight:
        lin = decoder.decoder.linears()
        layers = [(decoder.basis_mat.weight, None, "none"), (lin[0].weight, lin[0].bias, "relu"),
                  (lin[1].weight, lin[1].bias, "relu"), (lin[2].weight, lin[2].bias, "sigmoid")]
        # the two hidden layers' biases ride in the GEMMs: column 150 of the first (the expansion stage writes a one
        # there), column 128 of the second (its input gets a ones chunk behind the 128 activations: K = 144)
        hidden = lin[1].weight.shape[1]
        fold2 = lin[1].bias is not None and _pad16(hidden) + 16 <= MAX_K
        packed = PackedMLP(layers, in_width=RGB_IN_WIDTH, out_dim=3, pe_stage=True, dir_col=144,
                           k_override=[_pad16(decoder.basis_mat.weight.shape[1]), 160, _pad16(hidden) + (16 if fold2 else 0),
                                       _pad16(lin[2].weight.shape[1])],
                           bias_cols={1: 150, **({2: _pad16(hidden)} if fold2 else {})})
        decoder._lmb_packed = packed
    return packed


def rgb_backward_supported(decoder) -> bool:
    """The backward kernel is specialised to 27 basis outputs and two 128-wide hidden layers."""
    lin = decoder.decoder.linears()
    return (rgb_decoder_supported(decoder) and lin[0].weight.shape[0] == 128 and lin[1].weight.shape == (128, 128)
            and lin[2].weight.shape == (3, 128) and all(l.bias is not None for l in lin))


def rgb_decoder_backward(decoder, x: torch.Tensor, dout: torch.Tensor, count: Optional[torch.Tensor] = None,
                         zero_tail: bool = True):
    """One launch: ``dL/dx`` (bf16 ``[N, 160]``, feature columns filled) and the gradients of
    ``(basis.weight, lin0.weight, lin0.bias, lin1.weight, lin1.bias, lin2.weight, lin2.bias)``."""
    packed = _rgb_packed(decoder)
    packed.refresh()
    lib = native.lib()
    n_floats = int(lib.lmb_rgb_mlp_bwd_gbuf_floats())
    gbuf = torch.zeros(n_floats, device=x.device, dtype=torch.float32)
    dx = torch.zeros_like(x) if (count is not None and zero_tail) else torch.empty_like(x)
    dout = dout.contiguous().float()
    native.check(lib.lmb_rgb_mlp_bwd(x.data_ptr(), native.ptr(count), x.shape[0], packed.blob.data_ptr(), byref(packed.spec),
                                     dout.data_ptr(), dout.shape[1], dx.data_ptr(), gbuf.data_ptr(),
                                     packed.status.data_ptr(), native.stream_ptr()), "rgb_mlp_bwd")
    kf = decoder.basis_mat.weight.shape[1]
    o = 0
    g1 = gbuf[o:o + 128 * 160].view(128, 160); o += 128 * 160
    g2 = gbuf[o:o + 128 * 144].view(128, 144); o += 128 * 144
    g3t = gbuf[o:o + 128 * 16].view(128, 16); o += 128 * 16
    g0t = gbuf[o:o + 144 * 32].view(144, 32); o += 144 * 32
    db3 = gbuf[o:o + 16]
    grads = tuple(g.contiguous() for g in (g0t[:kf, :27].t(), g1[:, :150], g1[:, 150], g2[:, :128], g2[:, 128], g3t[:, :3].t(),
                                           db3[:3]))
    return dx, grads


class _RGBDecoderFn(torch.autograd.Function):
    """x: [N, 160] bf16 rows = [features(<=144), dir(3) at col 144, zeros]."""

    @staticmethod
    def forward(ctx, x, decoder, count, *params):
        ctx.decoder, ctx.count = decoder, count
        ctx.save_for_backward(x)
        return _rgb_packed(decoder).run(x, count)

    @staticmethod
    def backward(ctx, dout):
        (x,) = ctx.saved_tensors
        dec, count = ctx.decoder, ctx.count
        if rgb_backward_supported(dec):
            # rows past the device-side count are never read by the consumer of dx
            dx, grads = rgb_decoder_backward(dec, x, dout, count, zero_tail=False)
            lin = dec.decoder.linears()
            by_param = {id(dec.basis_mat.weight): grads[0], id(lin[0].weight): grads[1], id(lin[0].bias): grads[2],
                        id(lin[1].weight): grads[3], id(lin[1].bias): grads[4], id(lin[2].weight): grads[5],
                        id(lin[2].bias): grads[6]}
            params = list(dec.basis_mat.parameters()) + list(dec.decoder.parameters())
            return (dx, None, None, *[by_param.get(id(p)) for p in params])
        from ..components.fields.mlp_decoder import positional_encoding

        if count is not None:
            raise RuntimeError("colour head: a device-side row count needs the fused backward kernel (128-wide hidden layers)")

        with torch.enable_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            xin = x.detach().float().requires_grad_()
            kf = dec.basis_mat.weight.shape[1]
            f = dec.basis_mat(xin[:, :kf])
            d = xin[:, 144:147]
            mlp_in = torch.cat((f, d, positional_encoding(f.float(), 2), positional_encoding(d, 2)), dim=-1)
            out = dec.decoder.mlp(mlp_in).float()
            params = list(dec.basis_mat.parameters()) + list(dec.decoder.parameters())
            grads = torch.autograd.grad(out, [xin] + params, dout)
        return (grads[0].to(x.dtype), None, None, *grads[1:])


def rgb_decoder_forward(decoder, dirs: Optional[torch.Tensor], feats: torch.Tensor,
                        count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``feats``: either ``[N, 160]`` bf16 rows produced by ``vm_encode(out_width=160)`` or plain
    ``[N, C]`` features; ``dirs [N, 3]`` (``None``: the caller already wrote the direction columns).
    ``count``: device-side number of valid rows."""
    if feats.shape[1] == RGB_IN_WIDTH and feats.dtype == torch.bfloat16:
        x = feats
        if dirs is not None:
            x[:, 144:147] = dirs.to(torch.bfloat16)
    else:
        x = torch.cat((feats.to(torch.bfloat16), torch.zeros(feats.shape[0], 144 - feats.shape[1], device=feats.device,
                                                              dtype=torch.bfloat16),
                       dirs.to(torch.bfloat16),
                       torch.zeros(feats.shape[0], RGB_IN_WIDTH - 147, device=feats.device, dtype=torch.bfloat16)), dim=-1)
    params = list(decoder.basis_mat.parameters()) + list(decoder.decoder.parameters())
    if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in params)):
        return _RGBDecoderFn.apply(x.contiguous(), decoder, count, *params)
    return _rgb_packed(decoder).run(x.contiguous(), count)


# -- Scaffold / Octree anchor heads -------------------------------------------------------------------
def anchor_heads_supported(decoder, *inputs) -> bool:
    if not native.available():
        return False
    for seq in (decoder.mlp_opacity, decoder.mlp_cov, decoder.mlp_color):
        lin = [m for m in seq if isinstance(m, torch.nn.Linear)]
        if len(lin) != 2 or any(_pad16(l.weight.shape[0]) > MAX_N or _pad16(l.weight.shape[1]) > MAX_K for l in lin):
            return False
    return True


def _head_packed(decoder, name: str, seq, out_act: str) -> PackedMLP:
    key = f"_lmb_packed_{name}"
    lin = [m for m in seq if isinstance(m, torch.nn.Linear)]
    packed = getattr(decoder, key, None)
    if packed is None or packed.layers[0][0] is not lin[0].weight:
        packed = PackedMLP([(lin[0].weight, lin[0].bias, "relu"), (lin[1].weight, lin[1].bias, out_act)],
                           in_width=_pad16(lin[0].weight.shape[1]), out_dim=lin[1].weight.shape[0])
        setattr(decoder, key, packed)
    return packed


def anchor_heads_forward(decoder, op_in, cov_in, col_in):
    outs = []
    for name, seq, act, x in (("opacity", decoder.mlp_opacity, "tanh", op_in), ("cov", decoder.mlp_cov, "none", cov_in),
                              ("color", decoder.mlp_color, "sigmoid", col_in)):
        packed = _head_packed(decoder, name, seq, act)
        xb = torch.nn.functional.pad(x, (0, packed.in_width - x.shape[1])).to(torch.bfloat16).contiguous()
        outs.append(packed.run(xb))
    return tuple(outs)

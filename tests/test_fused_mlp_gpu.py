"""tcgen05 fused MLP kernel vs a plain PyTorch fp32 reference (bf16-rounded operands)."""
import pytest
import torch

from landmarksystem_b200.components.fields.mlp_decoder import MLPDecoder, positional_encoding
from landmarksystem_b200.models.gridnerf.gridnerf import RGBDecoder
from landmarksystem_b200.ops import fused_mlp

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf(t):
    return t.to(torch.bfloat16).float()


def _ref_mlp(dec, x):
    h = _bf(x)
    lin = dec.linears()
    for i, l in enumerate(lin):
        h = h @ _bf(l.weight).t() + (l.bias if l.bias is not None else 0)
        if i < len(lin) - 1:
            h = _bf(torch.relu(h))
    return dec.out_activation(h) if dec.out_activation is not None else h


@pytest.mark.parametrize("n", [1, 127, 128, 1000, 70000])
def test_generic_mlp_forward(n):
    torch.manual_seed(0)
    dec = MLPDecoder(inChanel=35, layer_width=64, num_layers=3, out_dim=7, out_activation=torch.nn.Sigmoid()).to(DEV)
    x = torch.randn(n, 35, device=DEV)
    assert fused_mlp.fused_mlp_supported(dec)
    with torch.no_grad():
        out = fused_mlp.mlp_forward(dec, x)
        ref = _ref_mlp(dec, x)
    dec._lmb_packed.check_status()
    assert out.shape == (n, 7)
    assert torch.allclose(out, ref, atol=2e-2), (out - ref).abs().max()


def test_generic_mlp_no_bias_tanh_and_backward():
    torch.manual_seed(0)
    dec = MLPDecoder(inChanel=32, layer_width=64, num_layers=2, out_dim=16, out_activation=torch.nn.Tanh(),
                     mlp_bias=False).to(DEV)
    x = torch.randn(777, 32, device=DEV, requires_grad=True)
    out = fused_mlp.mlp_forward(dec, x)
    ref = _ref_mlp(dec, x.detach())
    assert torch.allclose(out, ref, atol=2e-2)
    out.square().sum().backward()
    g_fused = dec.linears()[0].weight.grad.clone()
    dec.zero_grad()
    dec.mlp(x.detach()).square().sum().backward()
    g_ref = dec.linears()[0].weight.grad
    assert torch.allclose(g_fused, g_ref, atol=0.05 * g_ref.abs().max().item())


def test_rgb_decoder_forward_matches_module():
    torch.manual_seed(0)
    dec = RGBDecoder([48], [1, 2, 4], 27, view_pe=2, fea_pe=2, featureC=128).to(DEV)
    n = 5000
    feats = torch.randn(n, 144, device=DEV) * 0.3
    dirs = torch.nn.functional.normalize(torch.randn(n, 3, device=DEV), dim=-1)
    assert fused_mlp.rgb_decoder_supported(dec)
    with torch.no_grad():
        out = fused_mlp.rgb_decoder_forward(dec, dirs, feats)
        f = _bf(feats) @ _bf(dec.basis_mat.weight).t()
        d = _bf(dirs)
        x = torch.cat((f, d, positional_encoding(f, 2), positional_encoding(d, 2)), -1)
        ref = _ref_mlp(dec.decoder, x)
    dec._lmb_packed.check_status()
    assert torch.allclose(out, ref, atol=2e-2), (out - ref).abs().max()


def test_packed_weights_follow_fused_adam():
    """The fused optimiser writes parameters through raw pointers; the packed blob must still refresh."""
    from landmarksystem_b200.ops import FusedAdam

    torch.manual_seed(0)
    dec = MLPDecoder(inChanel=32, layer_width=64, num_layers=2, out_dim=16).to(DEV)
    opt = FusedAdam(dec.parameters(), lr=0.1)
    x = torch.randn(256, 32, device=DEV)
    with torch.no_grad():
        before = fused_mlp.mlp_forward(dec, x).clone()
    for p in dec.parameters():
        p.grad = torch.ones_like(p)
    opt.step()
    with torch.no_grad():
        after = fused_mlp.mlp_forward(dec, x)
        ref = _ref_mlp(dec, x)
    assert not torch.allclose(before, after, atol=1e-3)
    assert torch.allclose(after, ref, atol=2e-2)


@pytest.mark.parametrize("n_feat,n", [(144, 5000), (48, 333), (48, 40000)])
def test_rgb_decoder_backward_kernel(n_feat, n):
    """tcgen05 backward (recompute + dgrad + wgrad in one launch) vs fp32 autograd on bf16-rounded operands."""
    torch.manual_seed(0)
    dec = RGBDecoder([n_feat // 3], [1, 2, 4], 27, view_pe=2, fea_pe=2, featureC=128).to(DEV)
    with torch.no_grad():
        # hidden units sit firmly on one side of the relu (|bias| >> spread of the weighted sum): a unit whose
        # pre-activation is within rounding noise of zero would otherwise flip between the two implementations
        # and change that row's gradient by ~10 %
        for l in dec.decoder.linears()[:2]:
            l.weight.mul_(0.3)
            l.bias.copy_((torch.rand_like(l.bias) * 0.4 + 0.4) * torch.sign(torch.randn_like(l.bias)))
        dec.decoder.linears()[2].bias.uniform_(-0.2, 0.2)
    assert dec.basis_mat.weight.shape[1] == n_feat and fused_mlp.rgb_backward_supported(dec)
    feats = torch.randn(n, n_feat, device=DEV) * 0.3
    dirs = torch.nn.functional.normalize(torch.randn(n, 3, device=DEV), dim=-1)
    dout = torch.randn(n, 3, device=DEV)
    x = torch.zeros(n, fused_mlp.RGB_IN_WIDTH, device=DEV, dtype=torch.bfloat16)
    x[:, :n_feat] = feats.to(torch.bfloat16)
    x[:, 144:147] = dirs.to(torch.bfloat16)
    dx, grads = fused_mlp.rgb_decoder_backward(dec, x, dout)
    dec._lmb_packed.check_status()

    # plain fp32 PyTorch restatement with operands rounded to bf16 where the kernel keeps them in bf16
    # (activations x1/h1/h2 and the dz chain); accumulation in fp32
    lin = dec.decoder.linears()
    with torch.no_grad():
        W0 = _bf(dec.basis_mat.weight)
        W = [_bf(l.weight) for l in lin]
        b = [l.bias for l in lin]
        x0 = x[:, :n_feat].float()
        d = x[:, 144:147].float()
        f = _bf(x0 @ W0.t())
        s1, c1 = torch.sin(f), torch.cos(f)
        x1 = _bf(torch.cat((f, d, positional_encoding(f, 2), positional_encoding(d, 2)), -1))
        h1 = _bf(torch.relu(x1 @ W[0].t() + b[0]))
        h2 = _bf(torch.relu(h1 @ W[1].t() + b[1]))
        o = torch.sigmoid(h2 @ W[2].t() + b[2])
        dz3 = _bf(dout * o * (1 - o))
        dz2 = _bf((dz3 @ W[2]) * (h2 > 0))
        dz1 = _bf((dz2 @ W[1]) * (h1 > 0))
        dx1 = dz1 @ W[0]
        i = torch.arange(27, device=DEV)
        df = _bf(dx1[:, :27] + dx1[:, 30 + 2 * i] * c1 + dx1[:, 31 + 2 * i] * 2 * (1 - 2 * s1 * s1)
                 - dx1[:, 84 + 2 * i] * s1 - dx1[:, 85 + 2 * i] * 4 * s1 * c1)
        ref = (df @ W0, df.t() @ x0, dz1.t() @ x1, dz1.sum(0), dz2.t() @ h1, dz2.sum(0), dz3.t() @ h2, dz3.sum(0))

    def rel(a, b_):
        return float((a.float() - b_).norm() / (b_.norm() + 1e-12))

    errs = {"dx": rel(dx[:, :n_feat], ref[0])}
    for name, got, want in zip(("basis", "w1", "b1", "w2", "b2", "w3", "b3"), grads, ref[1:]):
        assert got.shape == want.shape, name
        errs[name] = rel(got, want)
    assert float(dx[:, n_feat:].float().abs().max()) == 0.0
    assert all(v < 1.5e-2 for v in errs.values()), errs


def test_rgb_decoder_backward_respects_count():
    torch.manual_seed(0)
    dec = RGBDecoder([16], [1, 2, 4], 27, view_pe=2, fea_pe=2, featureC=128).to(DEV)
    n, used = 1000, 300
    x = torch.zeros(n, fused_mlp.RGB_IN_WIDTH, device=DEV, dtype=torch.bfloat16)
    x[:, :48] = (torch.randn(n, 48, device=DEV) * 0.3).to(torch.bfloat16)
    x[used:] = float("nan")                       # rows past the count must not leak into any gradient
    dout = torch.randn(n, 3, device=DEV)
    count = torch.tensor([used], device=DEV, dtype=torch.int32)
    dx_c, g_c = fused_mlp.rgb_decoder_backward(dec, x, dout, count)
    dx_r, g_r = fused_mlp.rgb_decoder_backward(dec, x[:used].contiguous(), dout[:used].contiguous())
    dec._lmb_packed.check_status()
    assert torch.equal(dx_c[:used], dx_r) and float(dx_c[used:].float().abs().max()) == 0.0
    for a, b in zip(g_c, g_r):
        assert torch.isfinite(a).all() and torch.allclose(a, b, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("layers,in_dim,width,out_dim,act,bias,n", [
    (2, 32, 64, 16, None, False, 3000),                   # hash-grid density head: 32 -> 64 -> 1 + 15, no bias
    (3, 39, 64, 3, torch.nn.Sigmoid(), False, 70001),     # hash-grid colour head
    (3, 150, 128, 7, None, True, 515),                    # widest supported shape, with biases
])
def test_plain_mlp_backward_kernel(layers, in_dim, width, out_dim, act, bias, n):
    """Backward of plain relu networks in one tcgen05 launch (the colour-head kernel without its encoding stage) vs
    an fp32 PyTorch restatement with operands rounded to bf16 where the kernel keeps bf16."""
    torch.manual_seed(0)
    dec = MLPDecoder(inChanel=in_dim, layer_width=width, num_layers=layers, out_dim=out_dim, out_activation=act,
                     mlp_bias=bias).to(DEV)
    lin = dec.linears()
    with torch.no_grad():
        if bias:    # units firmly on one side of the relu, see test_rgb_decoder_backward_kernel
            for l in lin[:-1]:
                l.weight.mul_(0.3)
                l.bias.copy_((torch.rand_like(l.bias) * 0.4 + 0.4) * torch.sign(torch.randn_like(l.bias)))
    x = (torch.randn(n, in_dim, device=DEV) * 0.5).requires_grad_(True)
    dout = torch.randn(n, out_dim, device=DEV)
    out = fused_mlp.mlp_forward(dec, x)
    assert fused_mlp.mlp3_backward_supported(dec._lmb_packed)
    out.backward(dout)
    dec._lmb_packed.check_status()
    got = [x.grad.clone()] + [p.grad.clone() for l in lin for p in ((l.weight, l.bias) if bias else (l.weight,))]

    with torch.no_grad():
        W = [_bf(l.weight) for l in lin]
        b = [l.bias if bias else 0.0 for l in lin]
        hs = [_bf(x.detach())]
        for i in range(layers - 1):
            hs.append(_bf(torch.relu(hs[-1] @ W[i].t() + b[i])))
        z = hs[-1] @ W[-1].t() + b[-1]
        if act is not None:
            o = torch.sigmoid(z)
            dz = _bf(dout * o * (1 - o))
        else:
            dz = _bf(dout)
        want_rev = []
        for i in range(layers - 1, -1, -1):
            want_rev.append((dz.t() @ hs[i], dz.sum(0)))
            dh = dz @ W[i]
            dz = _bf(dh * (hs[i] > 0)) if i > 0 else dh
        want = [dz] + [t for wg, bg in reversed(want_rev) for t in ((wg, bg) if bias else (wg,))]

    def rel(a, b_):
        return float((a.float() - b_).norm() / (b_.norm() + 1e-12))

    errs = [rel(a, b_) for a, b_ in zip(got, want)]
    assert len(got) == len(want) and all(a.shape == b_.shape for a, b_ in zip(got, want))
    # without biases some units sit within rounding of the relu edge and may flip between the two computations
    assert all(e < (1.5e-2 if bias else 4e-2) for e in errs), errs

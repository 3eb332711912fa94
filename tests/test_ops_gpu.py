"""CUDA kernels vs their plain-PyTorch fp32 references (run on a B200)."""
import pytest
import torch

from landmarksystem_b200.ops import (FusedAdam, composite_render, composite_weights, vm_encode, vm_encode_reference)
from landmarksystem_b200.ops.composite import render_reference, weights_reference
from landmarksystem_b200.ops.hashgrid import hashgrid_encode, hashgrid_reference, make_meta

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _vm_case(B=3, C=16, L=2, N=5000, seed=0):
    g = torch.Generator().manual_seed(seed)
    planes = [torch.randn(B, 33 * (l + 1), 29 * (l + 1), C, generator=g) for l in range(L)]
    lines = [torch.randn(B, 17 * (l + 1), C, generator=g) for l in range(L)]
    coords = torch.rand(N, 4, generator=g) * 2.2 - 1.1          # some taps fall outside -> zero padding
    coords[:, 3] = torch.randint(-1, B + 1, (N,), generator=g).float()
    return planes, lines, coords


@pytest.mark.parametrize("C", [16, 48])
def test_vm_encode_fwd_bwd_fp32(C):
    planes, lines, coords = _vm_case(C=C)
    ref_p = [p.clone().requires_grad_() for p in planes]
    ref_l = [l.clone().requires_grad_() for l in lines]
    ref = vm_encode_reference(coords, ref_p, ref_l)
    gout = torch.randn(ref.shape, generator=torch.Generator().manual_seed(1))
    ref.backward(gout)
    cp = [p.to(DEV).requires_grad_() for p in planes]
    cl = [l.to(DEV).requires_grad_() for l in lines]
    out = vm_encode(coords.to(DEV), cp, cl)
    assert torch.allclose(out.cpu(), ref.detach(), atol=1e-5, rtol=1e-5)
    out.backward(gout.to(DEV))
    for a, b in zip(cp + cl, ref_p + ref_l):
        assert torch.allclose(a.grad.cpu(), b.grad, atol=2e-4, rtol=1e-4)


def test_vm_encode_bf16_shadow_and_sink():
    planes, lines, coords = _vm_case(C=16, L=1)
    cp = [torch.nn.Parameter(p.to(DEV)) for p in planes]
    cl = [torch.nn.Parameter(l.to(DEV)) for l in lines]
    for p in cp + cl:
        FusedAdam.attach_sink(p, shadow=True)
    out = vm_encode(coords.to(DEV), cp, cl, [p._lmb_shadow for p in cp], [l._lmb_shadow for l in cl])
    ref = vm_encode_reference(coords, [p.bfloat16().float() for p in planes], [l.bfloat16().float() for l in lines])
    assert torch.allclose(out.cpu(), ref, atol=1e-4, rtol=1e-4)
    out.sum().backward()
    assert cp[0].grad is None and cp[0]._lmb_grad_sink.abs().sum() > 0


def test_vm_encode_device_count():
    planes, lines, coords = _vm_case(C=16, L=1, N=1000)
    cp, cl = [p.to(DEV) for p in planes], [l.to(DEV) for l in lines]
    count = torch.tensor([300], device=DEV, dtype=torch.int32)
    out = vm_encode(coords.to(DEV), cp, cl, count=count)
    ref = vm_encode_reference(coords, planes, lines)
    assert torch.allclose(out[:300].cpu(), ref[:300], atol=1e-5) and out[300:].abs().sum() == 0


@pytest.mark.parametrize("S", [16, 64, 200])
def test_composite_fwd_bwd(S):
    torch.manual_seed(0)
    R = 257
    sigma = (torch.rand(R, S) * 4).requires_grad_()
    dists = torch.rand(R, S) * 0.3
    rgbs = torch.rand(R, S, 3).requires_grad_()
    z = torch.sort(torch.rand(R, S), -1)[0]
    w_ref, bg_ref = weights_reference(sigma, dists)
    rgb_ref, depth_ref, acc_ref = render_reference(w_ref, rgbs, z, 1.0)
    loss_ref = (rgb_ref * torch.arange(1, 4)).sum() + 0.3 * bg_ref.sum()
    loss_ref.backward()
    s2 = sigma.detach().to(DEV).requires_grad_()
    c2 = rgbs.detach().to(DEV).requires_grad_()
    w, bg = composite_weights(s2, dists.to(DEV))
    rgb, depth, acc = composite_render(w, c2, z.to(DEV), 1.0)
    assert torch.allclose(w.cpu(), w_ref, atol=1e-5) and torch.allclose(bg.cpu(), bg_ref, atol=1e-5)
    assert torch.allclose(rgb.cpu(), rgb_ref, atol=1e-4) and torch.allclose(depth.cpu(), depth_ref, atol=1e-4)
    loss = (rgb * torch.arange(1, 4, device=DEV)).sum() + 0.3 * bg.sum()
    loss.backward()
    assert torch.allclose(s2.grad.cpu(), sigma.grad, atol=2e-4, rtol=1e-3)
    assert torch.allclose(c2.grad.cpu(), rgbs.grad, atol=1e-5)


def test_fused_adam_matches_torch():
    torch.manual_seed(0)
    n = 4 * 1000 + 3
    a = torch.nn.Parameter(torch.randn(n, device=DEV))
    b = torch.nn.Parameter(a.detach().clone())
    FusedAdam.attach_sink(a, shadow=True)
    o1 = FusedAdam([a], lr=0.02, betas=(0.9, 0.99), eps=1e-8)
    o2 = torch.optim.Adam([b], lr=0.02, betas=(0.9, 0.99), eps=1e-8)
    for _ in range(5):
        g = torch.randn(n, device=DEV)
        a._lmb_grad_sink.copy_(g)
        b.grad = g.clone()
        o1.step(); o2.step()
        assert a._lmb_grad_sink.abs().sum() == 0          # cleared inside the kernel
    assert torch.allclose(a, b, atol=1e-5)
    assert torch.allclose(a._lmb_shadow.float(), a.detach().bfloat16().float())


@pytest.mark.parametrize("log2", [10, 19])
def test_hashgrid_fwd_bwd(log2):
    torch.manual_seed(0)
    meta = make_meta(8, 2, log2, 16, 1.6)
    table = torch.randn(meta.offsets[-1], 2) * 0.1
    x = torch.rand(3000, 3)
    t_ref = table.clone().requires_grad_()
    ref = hashgrid_reference(x, t_ref, meta)
    gout = torch.randn_like(ref)
    ref.backward(gout)
    t_gpu = table.to(DEV).requires_grad_()
    out = hashgrid_encode(x.to(DEV), t_gpu, meta)
    assert torch.allclose(out.cpu(), ref.detach(), atol=1e-5)
    out.backward(gout.to(DEV))
    assert torch.allclose(t_gpu.grad.cpu(), t_ref.grad, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("levels,features", [(8, 2), (6, 2), (5, 4), (16, 2)])
def test_hashgrid_on_ray_ordered_samples(levels, features):
    """Samples ordered along rays (neighbouring rows share cells on the coarse levels): the backward's in-warp sums over
    runs of equal cells, rows without a gradient in the middle of a run, a row count that is no multiple of the warp, and
    level counts that do and do not fill the 4-level groups."""
    g = torch.Generator().manual_seed(levels * 10 + features)
    meta = make_meta(levels, features, 14, 4, 1.7 if levels < 16 else 1.4)     # finest resolution stays below ~700 cells:
    # fp32 positions resolve the interpolation weights there whatever the rounding of x * scale + 0.5 (fused or not)
    table = torch.randn(meta.offsets[-1], features, generator=g) * 0.1
    R, S = 37, 53
    o = torch.rand(R, 1, 3, generator=g) * 0.3
    d = torch.nn.functional.normalize(torch.rand(R, 1, 3, generator=g), dim=-1)
    t = torch.linspace(0.0, 0.9, S)[None, :, None]
    x = (o + d * t).clamp(0.0, 1.0).reshape(-1, 3)
    gout = torch.randn(x.shape[0], levels * features, generator=g)
    gout[torch.rand(x.shape[0], generator=g) < 0.2] = 0.0
    t_ref = table.clone().requires_grad_()
    ref = hashgrid_reference(x, t_ref, meta)
    ref.backward(gout)
    t_gpu = table.to(DEV).requires_grad_()
    out = hashgrid_encode(x.to(DEV), t_gpu, meta)
    assert torch.allclose(out.cpu(), ref.detach(), atol=1e-5)
    out.backward(gout.to(DEV))
    assert torch.allclose(t_gpu.grad.cpu(), t_ref.grad, atol=2e-4, rtol=1e-4)


def test_lazy_adam_matches_dense_adam():
    """Deferred Adam on planes: fed the same gradients, the touched texels' shadows are current before every
    step and after a flush every parameter equals the dense fused Adam result."""
    torch.manual_seed(0)
    B, H, W, C = 2, 40, 36, 16
    plane0 = torch.randn(B, H, W, C, device=DEV) * 0.1
    dense = torch.nn.Parameter(plane0.clone())
    lazy = torch.nn.Parameter(plane0.clone())
    FusedAdam.attach_sink(dense, shadow=True)
    FusedAdam.attach_sink(lazy, shadow=True, lazy=True)
    opts = [FusedAdam([{"params": [p], "lr": 0.02, "lr_decay": 0.97}], betas=(0.9, 0.99), eps=1e-8) for p in (dense, lazy)]
    state = lazy._lmb_lazy
    g = torch.Generator(device=DEV).manual_seed(1)
    for it in range(14):
        # every step looks at a small random region, so most texels are skipped most of the time
        n = 300
        coords = torch.rand(n, 4, device=DEV, generator=g) * 0.5 - 1.0 + 1.5 * torch.rand(1, 4, device=DEV, generator=g)
        coords = coords.clamp(-1, 1)
        coords[:, 3] = torch.randint(0, B, (n,), device=DEV, generator=g).float()
        coords = coords.contiguous()
        state.prepare(lazy, coords)
        touched = state.need.view(B, H, W) != 0
        assert 0 < int(touched.sum()) < B * H * W
        # shadows of the texels about to be read are what a dense optimiser would hold
        assert torch.equal(lazy._lmb_shadow[touched], dense._lmb_shadow[touched]) or \
            (lazy._lmb_shadow[touched].float() - dense._lmb_shadow[touched].float()).abs().max() < 2e-3
        grad = torch.randn(B, H, W, C, device=DEV, generator=g) * touched[..., None]
        dense._lmb_grad_sink.copy_(grad)
        lazy._lmb_grad_sink.copy_(grad)
        for opt in opts:
            opt.step()
            opt.param_groups[0]["lr"] *= 0.97
        assert int(state.need.sum()) == 0
    assert state.last_step.min() < 14      # something was actually deferred
    state.flush(lazy)
    assert torch.allclose(lazy, dense, atol=2e-6, rtol=1e-5)
    assert (lazy._lmb_shadow.float() - dense._lmb_shadow.float()).abs().max() < 2e-3
    assert float(lazy._lmb_grad_sink.abs().max()) == 0.0


def test_lazy_adam_long_gap():
    """A texel left alone for hundreds of steps: the replay is cut off once beta1^k is below fp32 resolution
    and only decays the moments afterwards; the result still equals dense Adam."""
    torch.manual_seed(0)
    B, H, W, C = 1, 8, 8, 8
    p0 = torch.randn(B, H, W, C, device=DEV) * 0.1
    dense, lazy = torch.nn.Parameter(p0.clone()), torch.nn.Parameter(p0.clone())
    FusedAdam.attach_sink(dense, shadow=True)
    FusedAdam.attach_sink(lazy, shadow=True, lazy=True)
    opts = [FusedAdam([{"params": [p], "lr": 0.01, "lr_decay": 0.999}], betas=(0.9, 0.99), eps=1e-15) for p in (dense, lazy)]
    everywhere = torch.rand(4000, 4, device=DEV) * 2 - 1
    everywhere[:, 3] = 0
    corner = torch.tensor([[-1.0, -1.0, 0.0, 0.0]], device=DEV)
    g = torch.Generator(device=DEV).manual_seed(3)
    for it in range(420):
        coords = everywhere if it in (0, 1, 419) else corner
        lazy._lmb_lazy.prepare(lazy, coords.contiguous())
        touched = lazy._lmb_lazy.need.view(B, H, W) != 0
        grad = torch.randn(B, H, W, C, device=DEV, generator=g) * touched[..., None]
        if it == 419:
            assert (lazy._lmb_shadow.float() - dense._lmb_shadow.float()).abs().max() < 2e-3
        for p, opt in zip((dense, lazy), opts):
            p._lmb_grad_sink.copy_(grad)
            opt.step()
            opt.param_groups[0]["lr"] *= 0.999
    assert torch.allclose(lazy, dense, atol=5e-6, rtol=1e-5), (lazy - dense).abs().max()


@pytest.mark.parametrize("nonlinear,act", [(True, "softplus"), (True, "relu"), (False, "softplus")])
def test_vm_density_matches_reference(nonlinear, act):
    """Fused lookup + density head (forward, grid / line / weight gradients) vs the PyTorch restatement."""
    from landmarksystem_b200.ops.vm import vm_density, vm_density_reference

    torch.manual_seed(0)
    B, H, W, Z, C, L, n = 2, 24, 20, 16, 16, 2, 3000
    planes = [torch.nn.Parameter(torch.randn(B, H * (l + 1), W * (l + 1), C, device=DEV) * 0.3) for l in range(L)]
    lines = [torch.nn.Parameter(torch.randn(B, Z * (l + 1), C, device=DEV) * 0.3) for l in range(L)]
    weight = torch.nn.Parameter(torch.randn(1, L * C, device=DEV) * 0.3) if nonlinear else None
    coords = torch.rand(n, 4, device=DEV) * 2.2 - 1.1
    coords[:, 3] = torch.randint(-1, B, (n,), device=DEV).float()
    count = torch.tensor([n - 500], device=DEV, dtype=torch.int32)
    dsig = torch.randn(n, device=DEV)
    dsig[n - 500:] = 0
    shift = -0.5
    out = vm_density(coords, planes, lines, None, None, weight, nonlinear, act, shift, count)
    (out[: n - 500] * dsig[: n - 500]).sum().backward()
    got = [p.grad.clone() for p in planes + lines] + ([weight.grad.clone()] if nonlinear else [])
    for p in planes + lines + ([weight] if nonlinear else []):
        p.grad = None
    ref = vm_density_reference(coords[: n - 500], planes, lines, weight, nonlinear, act, shift)
    (ref * dsig[: n - 500]).sum().backward()
    want = [p.grad for p in planes + lines] + ([weight.grad] if nonlinear else [])
    assert torch.allclose(out[: n - 500], ref, atol=1e-5, rtol=1e-4)
    for g, w in zip(got, want):
        assert torch.allclose(g, w, atol=1e-4, rtol=1e-3), (g - w).abs().max()


@pytest.mark.parametrize("shape", [(3, 37, 53), (3, 128, 200), (1, 16, 16)])
def test_fused_l1_ssim_matches_conv_reference(shape):
    from landmarksystem_b200.components.utils import loss_utils
    from landmarksystem_b200.ops.ssim import fused_l1_ssim

    torch.manual_seed(0)
    img = torch.rand(*shape, device=DEV, requires_grad=True)
    gt = (img.detach() + 0.2 * torch.randn(*shape, device=DEV)).clamp(0, 1)
    l1, s = fused_l1_ssim(img, gt)
    (0.8 * l1 + 0.2 * (1 - s)).backward()
    got = img.grad.clone()
    img.grad = None
    # conv2d restatement on the CPU (the CUDA entry point of loss_utils.ssim dispatches to the fused kernel)
    x = img.detach().cpu().double().requires_grad_()
    g = gt.cpu().double()
    l1_ref = (x - g).abs().mean()
    s_ref = loss_utils.ssim(x, g)
    (0.8 * l1_ref + 0.2 * (1 - s_ref)).backward()
    assert abs(float(l1) - float(l1_ref)) < 1e-5 and abs(float(s) - float(s_ref)) < 1e-4
    assert torch.allclose(got.cpu().double(), x.grad, atol=2e-6, rtol=1e-3), (got.cpu().double() - x.grad).abs().max()


@pytest.mark.parametrize("B,n,det", [(62, 32, True), (126, 128, False), (509, 64, False), (1, 7, True)])
def test_pdf_resample_matches_torch(B, n, det):
    from landmarksystem_b200.components.ray_samplers import pdf_sampler
    from landmarksystem_b200.ops.pdf import pdf_resample

    torch.manual_seed(0)
    R = 300
    # bin widths between 0.5 and 1.5 units (bins far narrower than a float ulp of the position cannot be resolved)
    bins = 1.0 + torch.cumsum(0.5 + torch.rand(R, B + 1, device=DEV), -1) * (5.0 / (B + 1))
    weights = torch.rand(R, B, device=DEV) ** 4
    weights[::7] = 0                                      # rays without any mass fall back to the uniform PDF
    u = None if det else torch.rand(R, n, device=DEV)
    got = pdf_resample(bins, weights, n, u)
    # CPU statement of the same construction with the same uniform numbers
    w = weights.cpu().double() + 1e-5
    pdf = w / w.sum(-1, keepdim=True)
    cdf = torch.cat((torch.zeros(R, 1, dtype=torch.float64), pdf.cumsum(-1)), -1)
    uu = torch.linspace(0, 1, n, dtype=torch.float64).expand(R, n) if det else u.cpu().double()
    inds = torch.searchsorted(cdf, uu.contiguous(), right=True)
    below, above = (inds - 1).clamp(min=0), inds.clamp(max=B)
    c0, c1 = cdf.gather(-1, below), cdf.gather(-1, above)
    b0, b1 = bins.cpu().double().gather(-1, below), bins.cpu().double().gather(-1, above)
    den = torch.where(c1 - c0 < 1e-5, torch.ones_like(c0), c1 - c0)
    ref = b0 + (uu - c0) / den * (b1 - b0)
    # The inverse is ill-conditioned where the CDF is flat (bins without mass): a rounding-level change of u moves the
    # sample across such bins.  Positions therefore agree wherever the CDF has slope, and everywhere the CDF evaluated
    # at the returned position gives back u.
    pos = got.cpu().double()
    edges = bins.cpu().double()
    b = (torch.searchsorted(edges.contiguous(), pos.contiguous(), right=True) - 1).clamp(0, B - 1)
    e0, e1 = edges.gather(-1, b), edges.gather(-1, b + 1)
    f0, f1 = cdf.gather(-1, b), cdf.gather(-1, b + 1)
    back = f0 + (pos - e0) / (e1 - e0).clamp(min=1e-12) * (f1 - f0)
    assert (back - uu).abs().max() < 5e-4, (back - uu).abs().max()
    steep = (c1 - c0) > 1e-3
    assert ((pos - ref).abs()[steep]).max() < 1e-2
    assert torch.isfinite(got).all() and (got >= bins[:, :1] - 1e-4).all() and (got <= bins[:, -1:] + 1e-4).all()
    if det:
        assert (got[:, 1:] >= got[:, :-1] - 1e-5).all()
    assert pdf_sampler.sample_pdf(bins, weights, n, det=True).shape == (R, n)


def test_resize_nhwc_matches_interpolate():
    from landmarksystem_b200.ops.resize import resize_bilinear_nhwc, resize_linear_nlc

    torch.manual_seed(0)
    src = torch.randn(2, 13, 17, 16, device=DEV)
    for H2, W2 in ((29, 40), (13, 17), (5, 60), (1, 1)):
        got = resize_bilinear_nhwc(src, H2, W2)
        ref = torch.nn.functional.interpolate(src.permute(0, 3, 1, 2), size=(H2, W2), mode="bilinear", align_corners=True).permute(0, 2, 3, 1)
        assert got.shape == ref.shape and torch.allclose(got, ref, atol=1e-5), (H2, W2)
    line = torch.randn(3, 11, 48, device=DEV)
    got = resize_linear_nlc(line, 37)
    ref = torch.nn.functional.interpolate(line.permute(0, 2, 1), size=37, mode="linear", align_corners=True).permute(0, 2, 1)
    assert torch.allclose(got, ref, atol=1e-5)


def test_fused_adam_checkpoint_roundtrip_with_deferred_planes():
    """state_dict / load_state_dict carry the deferred-update moments: a restored optimiser continues exactly."""
    torch.manual_seed(0)

    def make():
        plane = torch.nn.Parameter(torch.randn(1, 16, 16, 8, device=DEV) * 0.1)
        w = torch.nn.Parameter(torch.randn(8, 8, device=DEV) * 0.1)
        FusedAdam.attach_sink(plane, shadow=True, lazy=True)
        return plane, w, FusedAdam([{"params": [plane], "lr": 0.02, "lr_decay": 0.99}, {"params": [w], "lr": 0.01, "lr_decay": 0.99}],
                                   capturable=True)

    def run(plane, w, opt, steps, seed):
        g = torch.Generator(device=DEV).manual_seed(seed)
        for _ in range(steps):
            coords = torch.rand(40, 4, device=DEV, generator=g) * 2 - 1
            coords[:, 3] = 0
            plane._lmb_lazy.prepare(plane, coords.contiguous())
            touched = plane._lmb_lazy.need.view(1, 16, 16) != 0
            plane._lmb_grad_sink.copy_(torch.randn(1, 16, 16, 8, device=DEV, generator=g) * touched[..., None])
            w.grad = torch.randn(8, 8, device=DEV, generator=g)
            opt.step()
            opt.zero_grad()

    a = make()
    torch.manual_seed(0)
    b = make()
    b[0].data.copy_(a[0].data); b[1].data.copy_(a[1].data)
    run(*a, 7, seed=1)
    sd = {k: (v if k != "state" else {i: {n: (t.clone() if torch.is_tensor(t) else t) for n, t in s.items()} for i, s in v.items()})
          for k, v in a[2].state_dict().items()}
    b[0].data.copy_(a[0].data); b[1].data.copy_(a[1].data); b[0]._lmb_shadow.copy_(a[0]._lmb_shadow)
    b[2].load_state_dict(sd)
    assert b[0]._lmb_lazy.steps_done == 7 and b[2].param_groups[0]["_dyn"].tolist()[1] == 8.0
    run(*a, 5, seed=2)
    run(*b, 5, seed=2)
    for x, y in ((a[0], b[0]), (a[1], b[1])):
        xs, ys = x, y
        if getattr(x, "_lmb_lazy", None) is not None:
            x._lmb_lazy.flush(x); y._lmb_lazy.flush(y)
        assert torch.allclose(xs, ys, atol=1e-6), (xs - ys).abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_vm_encode_sorted_backward_is_exact_and_reproducible(dtype):
    """Atomic-free backward: same gradients as the reduction-based kernel, and bit-identical from run to run."""
    from landmarksystem_b200.ops import vm

    torch.manual_seed(0)
    B, H, W, Z, C, L, n = 2, 21, 17, 9, 16, 2, 20000
    planes = [torch.nn.Parameter(torch.randn(B, H * (l + 1), W * (l + 1), C, device=DEV) * 0.3) for l in range(L)]
    lines = [torch.nn.Parameter(torch.randn(B, Z * (l + 1), C, device=DEV) * 0.3) for l in range(L)]
    coords = torch.rand(n, 4, device=DEV) * 2.4 - 1.2                 # some samples fall outside the grid
    coords[:, 3] = torch.randint(-1, B, (n,), device=DEV).float()
    coords[:50, :3] = torch.tensor([-1.0, 1.0, 0.3], device=DEV)       # exact grid corners / edges and long runs
    count = torch.tensor([n - 777], device=DEV, dtype=torch.int32)
    dout = torch.randn(n, L * C, device=DEV).to(dtype)
    shadows = None
    if dtype == torch.bfloat16:
        shadows = ([p.detach().to(dtype) for p in planes], [l.detach().to(dtype) for l in lines])

    def grads(flag):
        vm.DETERMINISTIC_BACKWARD = flag
        try:
            for p in planes + lines:
                p.grad = None
            out = vm.vm_encode(coords, planes, lines, *(shadows or (None, None)), count=count, out_dtype=dtype)
            out.backward(dout)
            return [p.grad.clone() for p in planes + lines]
        finally:
            vm.DETERMINISTIC_BACKWARD = False

    ref = grads(False)
    a = grads(True)
    b = grads(True)
    for x, y, r in zip(a, b, ref):
        assert torch.equal(x, y)                                       # reproducible to the bit
        assert torch.allclose(x, r, atol=2e-4, rtol=1e-3), (x - r).abs().max()


@pytest.mark.gpu
def test_fused_radam_matches_torch_radam():
    """Rectified Adam: the fused single-pass kernel follows torch.optim.RAdam through the unrectified first steps and
    the rectified ones (the switch happens at step 6 for beta2 = 0.999)."""
    from landmarksystem_b200.ops import FusedRAdam

    torch.manual_seed(0)
    w0 = torch.randn(1000, 37, device="cuda")
    a = torch.nn.Parameter(w0.clone()); b = torch.nn.Parameter(w0.clone())
    oa, ob = FusedRAdam([a], lr=1e-2, eps=1e-8), torch.optim.RAdam([b], lr=1e-2, eps=1e-8)
    for step in range(12):
        g = torch.randn_like(w0) * (0.1 + step)
        a.grad, b.grad = g.clone(), g.clone()
        oa.step(); ob.step()
        assert (a - b).abs().max().item() < 2e-6 * (1 + b.abs().max().item()), step


@pytest.mark.gpu
def test_ray_loss_kernels_match_the_pytorch_statements():
    """Distortion loss (both spellings) and the proposal inter-level loss: value and gradient against the plain
    PyTorch formulas on CPU in fp64-free fp32."""
    from landmarksystem_b200.components.utils import loss_utils as lu

    torch.manual_seed(0)
    R, S, E = 300, 48, 96
    edges = torch.sort(torch.rand(R, S + 1), dim=-1).values
    w = torch.rand(R, S) * 0.1
    m, d = (edges[:, 1:] + edges[:, :-1]) / 2, edges[:, 1:] - edges[:, :-1]
    # eff_distloss spelling
    wc = w.clone().requires_grad_(True)
    ref = lu.eff_distloss(wc, m, d); ref.backward()
    wg = w.cuda().requires_grad_(True)
    out = lu.eff_distloss(wg, m.cuda(), d.cuda()); out.backward()
    assert abs(out.item() - ref.item()) < 1e-5 * (1 + abs(ref.item()))
    assert (wg.grad.cpu() - wc.grad).abs().max().item() < 1e-6 + 1e-4 * wc.grad.abs().max().item()
    # nerfstudio spelling (S x S matrix on the CPU side)
    starts, ends = edges[:, :-1, None], edges[:, 1:, None]
    wc = w.clone().requires_grad_(True)
    ref = lu.distortion_loss([wc[..., None]], [starts], [ends]); ref.backward()
    wg = w.cuda().requires_grad_(True)
    out = lu.distortion_loss([wg[..., None]], [starts.cuda()], [ends.cuda()]); out.backward()
    assert abs(out.item() - ref.item()) < 1e-5 * (1 + abs(ref.item()))
    assert (wg.grad.cpu() - wc.grad).abs().max().item() < 1e-6 + 1e-4 * wc.grad.abs().max().item()
    # inter-level: proposal histogram on a coarser, unaligned partition
    env = torch.sort(torch.rand(R, E + 1), dim=-1).values
    env[:, 0], env[:, -1] = 0.0, 1.0
    w_env = torch.rand(R, E) * 0.05
    ec = w_env.clone().requires_grad_(True)
    ref = lu.interlevel_loss([ec[..., None], w[..., None]], [env[:, :-1, None], starts], [env[:, 1:, None], ends]); ref.backward()
    eg = w_env.cuda().requires_grad_(True)
    out = lu.interlevel_loss([eg[..., None], w.cuda()[..., None]], [env[:, :-1, None].cuda(), starts.cuda()],
                             [env[:, 1:, None].cuda(), ends.cuda()]); out.backward()
    assert abs(out.item() - ref.item()) < 1e-5 * (1 + abs(ref.item()))
    assert (eg.grad.cpu() - ec.grad).abs().max().item() < 1e-7 + 1e-4 * ec.grad.abs().max().item()


@pytest.mark.gpu
def test_proposal_resample_kernel_matches_the_pytorch_statement():
    """Histogram -> CDF -> inverse-CDF samples -> ordered merge with the existing edges, against the PyTorch chain
    (cumsum, searchsorted, gathers, concatenate + sort) of the same sampler."""
    from landmarksystem_b200.components.ray_samplers.proposal_network_sampler import PropPDFSampler
    from landmarksystem_b200.ops.pdf import prop_resample

    torch.manual_seed(0)
    R, E, n = 500, 96, 48
    existing = torch.sort(torch.rand(R, E + 1, device="cuda"), dim=-1).values
    weights = torch.rand(R, E, 1, device="cuda") ** 3
    weights[::7] = 0.0                                      # rays without any weight: the histogram is its padding
    for include in (True, False):
        s = PropPDFSampler(n, include_original=include)
        u = (torch.arange(n + 1, device="cuda") + torch.rand(R, n + 1, device="cuda")) / (n + 1)
        ref = s._resample_torch(weights, existing, u.contiguous(), 1e-5)
        out = prop_resample(weights[..., 0], existing, u, s.histogram_padding, 1e-5, include)
        assert out.shape == ref.shape
        assert (out[:, 1:] >= out[:, :-1]).all()
        assert (out - ref).abs().max().item() < 2e-5


@pytest.mark.gpu
def test_alpha_mask_pool_kernel_matches_max_pool3d():
    from landmarksystem_b200.ops.resize import alpha_mask_pool

    torch.manual_seed(0)
    alpha = torch.rand(37, 20, 51) ** 8 * 1.3                  # sparse, some values above 1 (clamped)
    alpha[:3] = 0; alpha[:, :2] = 0; alpha[..., 45:] = 0       # empty margins: the index box is a strict sub-box
    mask_ref, box_ref = alpha_mask_pool(alpha, 0.3)
    mask, box = alpha_mask_pool(alpha.cuda(), 0.3)
    assert torch.equal(mask.cpu(), mask_ref) and torch.equal(box.cpu(), box_ref)
    empty, box = alpha_mask_pool(torch.zeros(5, 6, 7, device="cuda"), 0.3)
    assert empty.sum() == 0 and box.tolist()[3:] == [-1, -1, -1]


@pytest.mark.gpu
def test_anchor_decode_epilogue_kernel_matches_the_indexing_path():
    """Scaffold-GS decoder at render time: the flag / scan / scatter kernels against the boolean-index path (same
    module in training mode under no_grad is not an option - it returns extra tensors - so the oracle is the CPU)."""
    from landmarksystem_b200.components.fields.anchor_decoder import AnchorDecoder

    torch.manual_seed(0)
    dec = AnchorDecoder(use_feat_bank=True, add_opacity_dist=False, add_color_dist=False, add_cov_dist=False, view_dim=3,
                        feat_dim=32, n_offsets=5).eval()
    n = 3000
    anchor, feat = torch.randn(n, 3), torch.randn(n, 32)
    offset, scaling = torch.randn(n, 5, 3) * 0.1, torch.rand(n, 6) + 0.1
    cam = torch.tensor([0.5, -4.0, 1.0])
    vis = torch.rand(n) > 0.3
    with torch.no_grad():
        ref = dec(cam, anchor, feat, offset, scaling, vis)
        dec_g = dec.cuda()
        out = dec_g(cam.cuda(), anchor.cuda(), feat.cuda(), offset.cuda(), scaling.cuda(), vis.cuda())
    assert out[5] is None and out[6] is None
    # candidates whose opacity is within rounding of zero may be kept on one side only: compare on the common set
    assert abs(out[0].shape[0] - ref[0].shape[0]) <= 3
    if out[0].shape[0] == ref[0].shape[0]:
        for a, b in zip(out[:5], ref[:5]):
            assert torch.allclose(a.cpu(), b, atol=2e-4, rtol=1e-3)


@pytest.mark.gpu
def test_segment_amax_kernel_matches_scatter_reduce():
    from landmarksystem_b200.components.fields.encodings.scaffoldgs_encoding import segment_amax

    torch.manual_seed(0)
    values = torch.randn(50000, 32) * 3
    index = torch.randint(0, 700, (50000,))
    index[index == 13] = 14                                  # an empty segment stays at -inf
    ref = segment_amax(values, index, 700)
    out = segment_amax(values.cuda(), index.cuda(), 700)
    assert torch.equal(out.cpu(), ref) and torch.isinf(ref[13]).all()


@pytest.mark.gpu
@pytest.mark.parametrize("hull", [False, True])
def test_fused_sampler_matches_the_unfused_front_end(hull):
    """Sampling distances, block-local coordinates and window-relative block ids from the one-kernel front end against
    ``UniformSampler.compute_z_vals`` + ``SceneManager.block_local_coords`` (dense spacing and render-time hull spacing)."""
    from landmarksystem_b200.components.ray_samplers import UniformSampler
    from landmarksystem_b200.components.scene import SceneManager
    from landmarksystem_b200.ops.sampler import uniform_sample_blocks
    from landmarksystem_b200.utils import Config

    g = torch.Generator().manual_seed(3)
    cfg = Config(lb=[0.0, 0.0, 0.0], ub=[200.0, 400.0, 30.0], plane_division=[2, 4], device=DEV)
    sm = SceneManager(cfg)
    sm.assign_local_block_partition([1, 2])
    sm.assign_relative_block_idx(1 * 4 + 1)
    R, S = 777, 48
    o = torch.stack((torch.rand(R, generator=g) * 200, torch.rand(R, generator=g) * 400, 80 + torch.rand(R, generator=g) * 20), -1)
    d = torch.nn.functional.normalize(torch.stack((torch.randn(R, generator=g) * 0.4, torch.randn(R, generator=g) * 0.4,
                                                   -torch.ones(R)), -1), dim=-1)
    d[:5, 2] = 0.3                                                   # a few rays look up: hull mode ends at `far`
    rays = torch.cat((o, d), -1).to(DEV)
    sampler = UniformSampler(num_samples=S, step_size=2.5, aabb=sm.aabb, near_far=[5.0, 300.0])
    z_ref = sampler.compute_z_vals(rays, S, False, hull)
    xyz = (rays[:, None, :3] + rays[:, None, 3:6] * z_ref[..., None]).reshape(-1, 3)
    inside = ~((xyz < sm.aabb[0]) | (xyz > sm.aabb[1])).any(-1)
    local, block = sm.block_local_coords(sm.normalize_coord(xyz))
    block = torch.where(inside, block, torch.full_like(block, -1.0))
    z, dists, xyzb, valid = uniform_sample_blocks(rays, S, sm.aabb, 5.0, 300.0, 2.5, sm._norm_lo, sm.aabb_norm_size, sm._partition,
                                                  (sm.relative_block_idx_x, sm.relative_block_idx_y),
                                                  tuple(sm.local_block_partition), None, hull=hull)
    torch.testing.assert_close(z, z_ref, rtol=1e-5, atol=1e-3)
    want_d = torch.cat((z_ref[:, 1:] - z_ref[:, :-1], torch.zeros_like(z_ref[:, :1])), -1)
    torch.testing.assert_close(dists, want_d, rtol=1e-4, atol=1e-3)
    # samples within a hair of a block or box face may land on the other side; everything else must agree exactly
    same = xyzb[:, 3] == block
    assert same.float().mean() > 0.999
    torch.testing.assert_close(xyzb[same][:, :3], local[same], rtol=1e-4, atol=1e-4)
    assert (valid == inside).float().mean() > 0.999


@pytest.mark.gpu
@pytest.mark.parametrize("C,tv_dev", [(16, True), (48, False)])
def test_adam_fused_with_plane_regularisers_matches_autograd_plus_adam(C, tv_dev):
    """Three optimiser steps on a channels-last plane whose TV and L1 terms are evaluated inside the Adam sweep (ping-pong
    parameter buffers) against the PyTorch statements of the two terms differentiated by autograd and ``torch.optim.Adam``;
    also the accumulated loss values, the bf16 shadow and that an ordinary ``.grad`` next to a sink is not dropped."""
    from landmarksystem_b200.components.fields.encodings.tensor_vm_encoding import tv_term

    g = torch.Generator(device=DEV).manual_seed(C)
    B, H, W = 2, 37, 53
    p0 = torch.randn(B, H, W, C, device=DEV, generator=g) * 0.1
    p0[0, 3, 4, :4] = 0.0                                          # sign(0) = 0 in the L1 gradient
    l1_w, tv_w0, decay, scale = 8e-5, 0.1, 0.9, 0.5
    data_grads = [torch.randn(B, H, W, C, device=DEV, generator=g) * 1e-3 for _ in range(3)]
    # reference: autograd of the statements + torch Adam
    ref = torch.nn.Parameter(p0.clone())
    ref_opt = torch.optim.Adam([ref], lr=0.02, betas=(0.9, 0.99), eps=1e-8)
    tv_w, want_vals = tv_w0, []
    for k in range(3):
        tv_w *= decay
        tv_val, l1_val = tv_w * tv_term(ref) * 1e-2, l1_w * ref.abs().mean()
        ((tv_val + l1_val) * scale).backward()
        ref.grad.add_(data_grads[k])
        ref_opt.step(); ref_opt.zero_grad()
        want_vals.append((float(tv_val), float(l1_val)))
    # fused path
    p = torch.nn.Parameter(p0.clone())
    FusedAdam.attach_sink(p, shadow=True)
    opt = FusedAdam([p], lr=0.02, betas=(0.9, 0.99), eps=1e-8)
    w_dev = torch.tensor([0.0, tv_w0], device=DEV)
    loss_out = torch.zeros(2, device=DEV)
    tv_host = tv_w0
    for k in range(3):
        w_dev.mul_(decay); tv_host *= decay
        FusedAdam.attach_plane_regulariser(p, w_dev if tv_dev else tv_host, 1, l1_w, scale, loss_out)
        loss_out.zero_()
        p._lmb_grad_sink.add_(data_grads[k] * 0.25)               # kernels' accumulator ...
        p.grad = data_grads[k] * 0.75                              # ... and an autograd gradient next to it
        opt.step()
        assert p.grad is None and float(p._lmb_grad_sink.abs().max()) == 0.0
        torch.testing.assert_close(loss_out.tolist(), list(want_vals[k]), rtol=2e-4, atol=1e-9)
    torch.testing.assert_close(p.data, ref.data, rtol=1e-4, atol=2e-6)
    torch.testing.assert_close(p._lmb_shadow.float(), p.data, rtol=1e-2, atol=1e-3)
    assert p._lmb_pong.data_ptr() != p.data.data_ptr()


@pytest.mark.parametrize("n", [1, 1023, 1024, 100003])
@pytest.mark.parametrize("offset", [0, 1])
def test_compact_rows_selects_every_masked_row_once(n, offset):
    """Mask compaction: the selected set, its count and the coordinates; rows of one 1024-element block stay in order.
    ``offset`` makes the mask start at an address that is not a multiple of four (the scalar mask-load path)."""
    from landmarksystem_b200.ops.select import compact_rows

    g = torch.Generator().manual_seed(n + offset)
    base = (torch.rand(n + offset, generator=g) < 0.3).to(DEV)
    mask = base[offset:]
    xyzb = torch.randn(n, 4, generator=g).to(DEV)
    idx, coords, count = compact_rows(mask, xyzb)
    k = int(count)
    want = mask.nonzero(as_tuple=True)[0]
    assert k == want.numel()
    got = idx[:k].long()
    assert torch.equal(got.sort().values, want)
    assert torch.equal(coords[:k], xyzb[got])
    same_block = (got[1:] // 1024) == (got[:-1] // 1024)
    assert bool((got[1:][same_block] > got[:-1][same_block]).all())


def test_vm_encode_writes_direction_tail():
    """The lookup kernel appends the ray direction of every row (and zeros) behind the features: bf16 rows of the colour
    head's width, with and without a row -> sample index, rows past the device-side count untouched."""
    planes, lines, coords = _vm_case(C=16, L=1, N=1000)
    cp, cl = [p.to(DEV) for p in planes], [l.to(DEV) for l in lines]
    S, R = 8, 125
    dirs = torch.randn(R, 3, device=DEV)
    idx = torch.randperm(R * S, device=DEV)[:1000].to(torch.int32)
    count = torch.tensor([700], device=DEV, dtype=torch.int32)
    width, col = 80, 48
    plain = vm_encode(coords.to(DEV), cp, cl, count=count, out_dtype=torch.bfloat16, out_width=width)
    for use_idx in (True, False):
        tail = (dirs if use_idx else dirs[idx.long() // S].contiguous(), idx if use_idx else None, S if use_idx else 1, col)
        out = vm_encode(coords.to(DEV), cp, cl, count=count, out_dtype=torch.bfloat16, out_width=width, tail=tail)
        assert torch.equal(out[:700, :col], plain[:700, :col])
        assert torch.equal(out[:700, col:col + 3], dirs[idx[:700].long() // S].to(torch.bfloat16))
        assert out[:700, col + 3:col + 16].abs().sum() == 0
        assert out[700:].abs().sum() == 0                  # zero_fill default: rows past the count stay zero

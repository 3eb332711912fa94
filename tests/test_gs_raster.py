"""Gaussian rasteriser: CPU oracle self-checks and CUDA kernels vs the oracle (forward and backward)."""
import math

import pytest
import torch

from landmarksystem_b200.components.data.cameras import Camera
from landmarksystem_b200.ops.gaussian_raster import GaussianRasterizationSettings, GaussianRasterizer
from landmarksystem_b200.synthetic import look_at


def _scene(n=60, W=48, H=32, seed=0, sh=True):
    g = torch.Generator().manual_seed(seed)
    means = (torch.rand(n, 3, generator=g) - 0.5) * torch.tensor([2.0, 1.4, 1.0])
    scales = torch.exp(torch.randn(n, 3, generator=g) * 0.3 - 2.2)
    rots = torch.nn.functional.normalize(torch.randn(n, 4, generator=g), dim=-1)
    opac = torch.sigmoid(torch.randn(n, 1, generator=g))
    shs = torch.randn(n, 16, 3, generator=g) * 0.2 if sh else None
    cols = None if sh else torch.rand(n, 3, generator=g)
    c2w = look_at(torch.tensor([0.3, -0.2, 3.0]), torch.zeros(3), up=(0.0, 1.0, 0.0)).numpy()
    cam = Camera.from_c2w(c2w, W, H, focal_x=40.0)
    s = GaussianRasterizationSettings(H, W, cam.tanfovx, cam.tanfovy, torch.tensor([0.1, 0.2, 0.3]), 1.0,
                                      cam.world_view_transform, cam.full_proj_transform, 3 if sh else 0, cam.camera_center)
    return means, scales, rots, opac, shs, cols, s


def test_reference_renders_something_and_is_differentiable():
    means, scales, rots, opac, shs, cols, s = _scene(n=20)
    means.requires_grad_()
    img, radii, alpha = GaussianRasterizer(s)(means, None, opac, shs=shs, scales=scales, rotations=rots)
    assert img.shape == (3, 32, 48) and (radii > 0).sum() > 5 and alpha.max() > 0.1
    img.sum().backward()
    assert torch.isfinite(means.grad).all() and means.grad.abs().sum() > 0


@pytest.mark.gpu
@pytest.mark.parametrize("sh", [True, False])
def test_cuda_matches_reference_forward_backward(sh):
    means, scales, rots, opac, shs, cols, s = _scene(sh=sh)
    leaves_c = [t.clone().requires_grad_() for t in (means, scales, rots, opac, shs if sh else cols)]
    mc, sc, rc, oc, cc = leaves_c
    img_ref, radii_ref, _ = GaussianRasterizer(s)(mc, None, oc, shs=cc if sh else None, colors_precomp=None if sh else cc,
                                                   scales=sc, rotations=rc)
    w = torch.rand(3, s.image_height, s.image_width, generator=torch.Generator().manual_seed(1))
    (img_ref * w).sum().backward()
    leaves_g = [t.clone().cuda().requires_grad_() for t in (means, scales, rots, opac, shs if sh else cols)]
    mg, sg, rg, og, cg = leaves_g
    img, radii, _ = GaussianRasterizer(s)(mg, None, og, shs=cg if sh else None, colors_precomp=None if sh else cg,
                                           scales=sg, rotations=rg)
    assert torch.equal(radii.cpu(), radii_ref)
    assert torch.allclose(img.cpu(), img_ref, atol=2e-4), (img.cpu() - img_ref).abs().max()
    (img * w.cuda()).sum().backward()
    for name, a, b in zip(("means", "scales", "rots", "opacity", "colour"), leaves_g, leaves_c):
        scale = b.grad.abs().max().item() + 1e-8
        assert torch.allclose(a.grad.cpu(), b.grad, atol=2e-3 * scale + 1e-6, rtol=1e-2), (name, (a.grad.cpu() - b.grad).abs().max(), scale)


@pytest.mark.gpu
def test_visible_filter_matches_radii():
    means, scales, rots, opac, shs, cols, s = _scene(n=500)
    r_cpu = GaussianRasterizer(s).visible_filter(means, scales, rots)
    r_gpu = GaussianRasterizer(s).visible_filter(means.cuda(), scales.cuda(), rots.cuda())
    assert torch.equal(r_cpu, r_gpu.cpu())


@pytest.mark.gpu
def test_radix_sort_and_scan():
    from landmarksystem_b200.ops import native
    from landmarksystem_b200.ops.gaussian_raster import _lib_ll

    torch.manual_seed(0)
    n = 300_000
    keys = torch.randint(0, 2 ** 44, (n,), dtype=torch.int64, device="cuda")
    vals = torch.arange(n, dtype=torch.int32, device="cuda")
    ref_keys, order = torch.sort(keys, stable=True)
    ws = torch.empty(_lib_ll("lmb_radix_sort_scratch_bytes")(n), dtype=torch.uint8, device="cuda")
    native.check(native.lib().lmb_radix_sort_pairs(keys.data_ptr(), vals.data_ptr(), None, n, 0, 48, ws.data_ptr(),
                                                   native.stream_ptr()), "sort")
    assert torch.equal(keys, ref_keys) and torch.equal(vals.long(), order)
    x = torch.randint(0, 50, (n,), dtype=torch.int32, device="cuda")
    out = torch.empty_like(x)
    ws2 = torch.empty(_lib_ll("lmb_scan_scratch_bytes")(n), dtype=torch.uint8, device="cuda")
    native.check(native.lib().lmb_exclusive_scan_u32(x.data_ptr(), out.data_ptr(), n, ws2.data_ptr(), native.stream_ptr()), "scan")
    assert torch.equal(out.long(), torch.cumsum(x.long(), 0) - x.long())


def test_baseline_restatement_agrees_with_the_oracle():
    """The PyTorch restatement timed as the 3DGS baseline (``baseline/gs_restatement.py``, written independently of the
    oracle in ``ops/gaussian_raster.py``) renders the same image from the same parameters."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from baseline.gs_restatement import render

    means, scales, rots, opac, shs, _, s = _scene(n=80)
    want, _, _ = GaussianRasterizer(s)(means, None, opac, shs=shs, scales=scales, rotations=rots)
    got = render(means, scales.log(), rots, torch.logit(opac), shs, s.viewmatrix, s.projmatrix, s.campos, s.image_width,
                 s.image_height, s.tanfovx, s.tanfovy, s.bg)
    assert got.shape == want.shape
    assert float((got - want).abs().max()) < 2e-3, float((got - want).abs().max())


def test_baseline_orbit_camera_equals_the_framework_camera():
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    from baseline.gs_restatement import orbit_camera

    for k in (0, 7, 123):
        cam = bench.gs_orbit_camera(k, "cpu")
        view, proj, campos, tanx, tany = orbit_camera(k, "cpu")
        torch.testing.assert_close(view, cam.world_view_transform, rtol=1e-4, atol=1e-3)
        torch.testing.assert_close(proj, cam.full_proj_transform, rtol=1e-4, atol=1e-3)
        torch.testing.assert_close(campos, cam.camera_center, rtol=1e-5, atol=1e-3)
        assert abs(tanx - cam.tanfovx) < 1e-6 and abs(tany - cam.tanfovy) < 1e-6

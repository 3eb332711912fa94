"""Per-sample glue kernels of the hash-grid fields (``ops/csrc/ngp_field.cu``) against their PyTorch statements."""
import pytest
import torch

from landmarksystem_b200.components.utils.sh_utils import sh_basis
from landmarksystem_b200.ops import ngp_field

cuda = pytest.mark.gpu


def _rays(R, dev, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    o = (torch.rand(R, 3, generator=g) * 0.6 + 0.2).to(dev)
    d = torch.nn.functional.normalize(torch.randn(R, 3, generator=g), dim=-1).to(dev) * 1.7   # not unit on purpose
    return o, d


def test_cpu_paths_use_the_pytorch_statements():
    d = torch.nn.functional.normalize(torch.randn(50, 3), dim=-1)
    assert torch.equal(ngp_field.sh_encode((d + 1) / 2, 4, True), sh_basis(((d + 1) / 2) * 2 - 1, 3))
    R, S, G, A = 6, 5, 15, 8
    o, dv = _rays(R, "cpu")
    h = torch.randn(R * S, 1 + G, requires_grad=True)
    app = torch.randn(R, A, requires_grad=True)
    inside = torch.rand(R * S) > 0.2
    rows, sigma = ngp_field.head_rows(None, S, dv, h, inside, app, A, 48)
    assert rows.shape == (R * S, 48) and rows.dtype == torch.bfloat16 and sigma.shape == (R * S,)
    (rows.float().sum() + sigma.sum()).backward()
    assert h.grad is not None and app.grad is not None
    assert torch.allclose(app.grad, torch.full_like(app.grad, float(S)))


@cuda
@pytest.mark.parametrize("levels", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("unit_range", [True, False])
def test_sh_encode_kernel(levels, unit_range):
    dev = "cuda"
    d = torch.nn.functional.normalize(torch.randn(10007, 3, device=dev), dim=-1)
    x = (d + 1) / 2 if unit_range else d
    got = ngp_field.sh_encode(x, levels, unit_range)
    want = sh_basis((x * 2 - 1) if unit_range else x, levels - 1)
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=2e-6, rtol=1e-5)


@cuda
@pytest.mark.parametrize("division,only_block", [((1, 1), -1), ((2, 2), -1), ((2, 3), 4)])
@pytest.mark.parametrize("subset", [False, True])
def test_sample_positions_kernel(division, only_block, subset):
    dev = "cuda"
    R, S = 301, 17
    o, dv = _rays(R, dev)
    z = torch.rand(R * S, device=dev) * 0.6
    aabb = torch.tensor([[0.05, 0.1, 0.0], [0.95, 1.0, 0.9]], device=dev)
    idx = (torch.rand(R * S, device=dev) > 0.4).nonzero(as_tuple=True)[0] if subset else None
    nx, ny = division
    got_x, got_in = ngp_field.sample_positions(idx, S, o, dv, z, aabb, aabb.reshape(-1).tolist(), nx, ny, only_block)
    want_x, want_in = ngp_field.positions_reference(idx, S, o, dv, z, aabb, nx, ny, only_block)
    # a sample within rounding distance of a wall may flip its flag between the two evaluation orders
    agree = got_in == want_in
    assert agree.float().mean() > 0.999
    assert torch.allclose(got_x[agree], want_x[agree], atol=2e-5)


@cuda
@pytest.mark.parametrize("subset", [False, True])
@pytest.mark.parametrize("with_app", [True, False])
@pytest.mark.parametrize("A,W", [(8, 48), (32, 64), (5, 40)])
def test_head_rows_kernel_forward_and_backward(subset, with_app, A, W):
    dev = "cuda"
    R, S, G = 257, 19, 15
    _, dv = _rays(R, dev)
    idx = (torch.rand(R * S, device=dev) > 0.3).nonzero(as_tuple=True)[0] if subset else None
    M = idx.numel() if subset else R * S
    h0 = torch.randn(M, 1 + G, device=dev)
    h0[:7, 0] = torch.tensor([-30.0, 30.0, 16.0, -16.0, 0.0, 14.9, -14.9], device=dev)[: min(7, M)]
    app0 = torch.randn(R, A, device=dev)
    inside = torch.rand(M, device=dev) > 0.15
    wr = torch.randn(M, W, device=dev)
    ws = torch.randn(M, device=dev)

    def run(fn):
        h = h0.clone().requires_grad_()
        app = app0.clone().requires_grad_() if with_app else None
        rows, sigma = fn(idx, S, dv, h, inside, app, A, W) if fn is ngp_field.head_rows else fn(idx, S, dv, h, inside, app, W)
        loss = (rows.float() * wr).sum() + (sigma * ws).sum()
        loss.backward()
        return rows, sigma, h.grad, None if app is None else app.grad

    got = run(ngp_field.head_rows)
    want = run(ngp_field.head_rows_reference)
    assert torch.equal(got[0][:, 16:], want[0][:, 16:])                       # copies and zero tail: exact
    assert torch.allclose(got[0][:, :16].float(), want[0][:, :16].float(), atol=8e-3)   # SH in bf16
    assert torch.allclose(got[1], want[1], rtol=1e-5, atol=1e-6)
    assert torch.allclose(got[2][:, 1:], want[2][:, 1:], atol=1e-6)          # geometry columns: bf16 gradient, masked
    assert torch.allclose(got[2][:, 0], want[2][:, 0], rtol=1e-5, atol=1e-6)  # exp(clamp(h0)) * d_sigma * inside
    if with_app:
        assert torch.allclose(got[3], want[3], rtol=1e-4, atol=1e-4)


@cuda
def test_occupancy_refresh_kernels():
    dev = "cuda"
    res, level = 16, 1
    n_cells = res ** 3
    roi = [-1.0, -2.0, 0.0, 1.0, 2.0, 3.0]
    occs = torch.rand(n_cells, device=dev)
    before = occs.clone()
    idx = torch.cat((torch.randint(n_cells, (900,), device=dev), torch.arange(40, device=dev), torch.arange(40, device=dev)))
    xyz, decayed = ngp_field.occ_cells(idx, n_cells, res, roi, level, 1234, True, occs, 0.95)
    assert torch.allclose(decayed, before[idx] * 0.95)
    # every position lies inside its cell of the cascade (region scaled by 2^level about the centre)
    lo, hi = torch.tensor(roi[:3], device=dev), torch.tensor(roi[3:], device=dev)
    centre, half = 0.5 * (lo + hi), 0.5 * (hi - lo) * 2.0
    u = ((xyz - centre) / half * 0.5 + 0.5) * res
    cell = torch.stack((idx // (res * res), (idx // res) % res, idx % res), -1).float()
    assert bool(((u >= cell - 1e-4) & (u <= cell + 1 + 1e-4)).all())
    assert float((u - cell).std()) > 0.2                        # jittered, not cell centres
    fresh = torch.rand(idx.numel(), device=dev) * 1.5
    ngp_field.occ_update(idx, decayed, fresh, occs)
    want = before.clone()
    want[idx] = before[idx] * 0.95
    want = want.scatter_reduce(0, idx, fresh, reduce="amax", include_self=True)
    assert torch.allclose(occs, want)
    untouched = torch.ones(n_cells, dtype=torch.bool, device=dev)
    untouched[idx] = False
    assert torch.equal(occs[untouched], before[untouched])
    # all cells (idx None), no jitter: cell centres
    xyz_all, _ = ngp_field.occ_cells(None, n_cells, res, roi, 0, 1, False, occs, 1.0)
    c0 = torch.tensor([0.5, 0.5, 0.5], device=dev) / res
    assert torch.allclose(xyz_all[0], lo + c0 * (hi - lo), atol=1e-5)
    binaries = torch.zeros(n_cells, dtype=torch.bool, device=dev)
    scratch = torch.zeros(1, dtype=torch.float64, device=dev)
    for thre in (0.01, 10.0):
        ngp_field.occ_binarise(occs, thre, binaries.view(torch.uint8), scratch)
        assert torch.equal(binaries, occs > min(float(occs.double().mean()), thre))


@cuda
def test_occ_cull_kernel_matches_the_tensor_statement():
    dev = "cuda"
    R, S = 333, 70
    g = torch.Generator().manual_seed(3)
    counts = torch.randint(0, S + 1, (R,), generator=g).to(torch.int32).to(dev)
    counts[:3] = torch.tensor([0, S, 1], dtype=torch.int32)
    valid = torch.arange(S, device=dev)[None] < counts[:, None]
    ts = (torch.rand(R, S, generator=g).to(dev).cumsum(1) * 0.05) * valid
    te = (ts + 0.04) * valid
    sigma = (torch.rand(R, S, generator=g).to(dev) ** 3 * 40.0) * valid
    thre, eps = 0.05, 1e-3
    alpha = 1.0 - torch.exp(-sigma * (te - ts))
    trans = torch.cumprod(torch.cat((torch.ones_like(alpha[:, :1]), 1.0 - alpha), -1), -1)[:, :-1]
    keep = valid & (alpha >= thre) & (trans >= eps)
    near = ((alpha - thre).abs() < 1e-5) | ((trans - eps).abs() < 1e-6)        # decisions within rounding of a threshold
    order = torch.argsort((~keep).to(torch.int8), dim=1, stable=True)
    want_ts, want_te = torch.gather(ts, 1, order), torch.gather(te, 1, order)
    want_counts = keep.sum(1).to(torch.int32)
    got_ts, got_te, got_counts = ts.clone(), te.clone(), counts.clone()
    ngp_field.occ_cull(sigma.contiguous(), got_ts, got_te, got_counts, thre, eps)
    clean = ~(near & valid).any(1)
    assert clean.float().mean() > 0.9
    assert torch.equal(got_counts[clean], want_counts[clean])
    front = torch.arange(S, device=dev)[None] < want_counts[:, None]
    sel = front & clean[:, None]
    assert torch.equal(got_ts[sel], want_ts[sel]) and torch.equal(got_te[sel], want_te[sel])
    assert float(got_ts[~front & clean[:, None]].abs().sum()) == 0.0


@cuda
@pytest.mark.parametrize("subset", [False, True])
def test_gather_cached_rows_kernel(subset):
    dev = "cuda"
    R, S = 97, 40
    g = torch.Generator().manual_seed(5)
    source = torch.stack([torch.randperm(S, generator=g) for _ in range(R)]).to(torch.int32).to(dev)
    n_rows = R * S
    where = None
    if subset:
        where = torch.randint(0, n_rows, (R * S,), generator=g).to(dev)
    a = torch.randn(n_rows, 32, generator=g).to(torch.bfloat16).to(dev)
    b = torch.randn(n_rows, 16, generator=g).to(dev)
    idx = (torch.rand(R * S, generator=g) < 0.5).nonzero(as_tuple=True)[0].to(dev)
    got_a, got_b = ngp_field.gather_cached_rows(idx, S, source, where, a, b)
    before = (idx // S) * S + source.reshape(-1)[idx].long()
    rows = before if where is None else where[before]
    assert torch.equal(got_a, a[rows]) and torch.equal(got_b, b[rows])

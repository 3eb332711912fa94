"""InstantNGP / Nerfacto: occupancy marching, proposal sampling, scene contraction and short trainings."""
import os

import numpy as np
import pytest
import torch

from landmarksystem_b200.components.ray_samplers.proposal_network_sampler import (PropPDFSampler, SpacedSampler,
                                                                                  spacing_fn, spacing_fn_inv)
from landmarksystem_b200.configs import BaseConfig
from landmarksystem_b200.models.nerfacto.nerfacto import scene_contraction
from landmarksystem_b200.ops.occgrid import OccGridEstimator

ROOT = os.path.join(os.path.dirname(__file__), "..", "landmarksystem_b200", "models")


def _grid(levels=2, res=8, seed=0):
    est = OccGridEstimator([-1.0, -1, -1, 1, 1, 1], res, levels)
    g = torch.Generator().manual_seed(seed)
    est.binaries = torch.rand(levels, res, res, res, generator=g) > 0.6
    return est


def _rays(n=64, seed=1):
    g = torch.Generator().manual_seed(seed)
    o = torch.tensor([0.0, 0.0, 3.0]) + 0.3 * torch.randn(n, 3, generator=g)
    d = torch.nn.functional.normalize(-o + 0.8 * torch.randn(n, 3, generator=g), dim=-1)
    return o, d


def test_march_reference_samples_lie_in_occupied_cells():
    est = _grid(levels=1)
    o, d = _rays(16)
    counts, ts, te = est.sampling(o, d, near_plane=0.1, far_plane=10.0, render_step_size=0.05, max_samples=64)
    assert counts.sum() > 0
    for r in range(16):
        for s in range(int(counts[r])):
            p = o[r] + d[r] * 0.5 * (ts[r, s] + te[r, s])
            idx = ((p * 0.5 + 0.5) * 8).long().clamp(0, 7)
            assert est.binaries[0, idx[0], idx[1], idx[2]]
            assert abs(float(te[r, s] - ts[r, s]) - 0.05) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("cone", [0.0, 0.01])
def test_march_kernel_matches_reference(cone):
    est = _grid(levels=2)
    o, d = _rays(200)
    c0, ts0, te0 = est.sampling(o, d, near_plane=0.1, far_plane=10.0, render_step_size=0.04, cone_angle=cone, max_samples=96)
    est_g = _grid(levels=2).cuda()
    c1, ts1, te1 = est_g.sampling(o.cuda(), d.cuda(), near_plane=0.1, far_plane=10.0, render_step_size=0.04, cone_angle=cone,
                                  max_samples=96)
    same = (c0 == c1.cpu())
    assert same.float().mean() > 0.97          # fp rounding at cell borders may flip isolated samples
    rows = same.nonzero().squeeze(-1)
    assert torch.allclose(ts0[rows], ts1.cpu()[rows], atol=1e-3)


def test_grid_update_marks_dense_region():
    est = OccGridEstimator([-1.0, -1, -1, 1, 1, 1], 16, 1)
    est.train()
    est.update_every_n_steps(0, lambda x: (x.norm(dim=-1) < 0.5).float(), occ_thre=0.01)
    frac = est.binaries.float().mean()
    assert 0.02 < frac < 0.2                   # ~ volume of the radius-0.5 ball inside the cube
    assert est.binaries[0, 8, 8, 8] and not est.binaries[0, 0, 0, 0]


def test_spacing_and_pdf_sampler():
    x = torch.tensor([0.1, 0.9, 1.0, 3.0, 50.0])
    assert torch.allclose(spacing_fn_inv(spacing_fn(x)), x, rtol=1e-5)
    sp = SpacedSampler().eval()
    o, d = _rays(8)
    rs = sp(o, d, 0.5, 20.0, 32)
    assert rs.starts.shape == (8, 32, 1) and torch.all(rs.ends >= rs.starts)
    assert abs(float(rs.starts[0, 0, 0]) - 0.5) < 1e-4 and abs(float(rs.ends[0, -1, 0]) - 20.0) < 1e-3
    w = torch.zeros(8, 32, 1)
    w[:, 10:12] = 1.0
    fine = PropPDFSampler(include_original=False).eval()(rs, w, 16)
    inside = (fine.spacing_starts[..., 0] >= rs.spacing_starts[:, 9:10, 0]) & (fine.spacing_ends[..., 0] <= rs.spacing_ends[:, 12:13, 0])
    assert inside.float().mean() > 0.8         # resampled intervals concentrate where the weight is


def test_scene_contraction():
    x = torch.tensor([[0.5, -0.2, 0.1], [4.0, 0.0, 0.0], [0.0, -100.0, 50.0]])
    y = scene_contraction(x)
    assert torch.allclose(y[0], x[0]) and torch.allclose(y[1], torch.tensor([1.75, 0.0, 0.0]))
    assert y.abs().max() < 2.0


@pytest.mark.parametrize("family,module,cls", [("instant_ngp", "instant_ngp_trainer", "NGPTrainer"),
                                                ("nerfacto", "nerfacto_trainer", "NerfactoTrainer")])
def test_cpu_smoke(family, module, cls, tmp_path):
    import importlib

    mod = importlib.import_module(f"landmarksystem_b200.models.{family}.{module}")
    cfg = BaseConfig.from_file(os.path.join(ROOT, family, "confs", "synthetic_tiny.py"),
                               {"basedir": str(tmp_path), "device": "cpu", "n_iters": "3", "datadir": "ring:3:12x12:14:3",
                                "batch_size": "64", "progress_refresh_rate": "100"})
    trainer = getattr(mod, cls)(cfg)
    trainer.train()
    assert os.path.exists(os.path.join(trainer.logfolder, "state_dict.th"))
    state = torch.load(os.path.join(trainer.logfolder, "state_dict.th"), weights_only=False)
    assert "mlp_base_grid.tcnn_encoding.params" in state      # reference checkpoint key of the hash table
    # helper methods of the reference's trainers / models
    trainer.iteration = 10
    lr = trainer.update_learning_rate()
    assert lr == trainer.lr_at(10) and all(g["lr"] == lr for g in trainer.optimizer.param_groups if g.get("scheduled", True))
    trainer.save_optimizer(str(tmp_path / "opt.th"))
    assert "optimizer" in torch.load(str(tmp_path / "opt.th"), weights_only=False)
    if family == "nerfacto":
        m = trainer.module
        pts = torch.rand(5, 7, 3) * 2 - 1
        with torch.no_grad():
            assert m.density_fn(pts).shape == (5, 7, 1)
            assert m.proposal_networks.get_density(pts.reshape(-1, 3), 1).shape[0] == 35
        assert m.proposal_sampler is m.sampler
        m.step_cb(7)
        assert m.sampler._step == 7
        half = m.set_anneal(cfg.proposal_weights_anneal_max_num_iters // 2)
        b = cfg.proposal_weights_anneal_slope
        assert abs(half - b * 0.5 / ((b - 1) * 0.5 + 1)) < 1e-9 and m.sampler._anneal == half and m.set_anneal(10 ** 9) == 1.0


@pytest.mark.gpu
@pytest.mark.parametrize("family,module,cls", [("instant_ngp", "instant_ngp_trainer", "NGPTrainer"),
                                                ("nerfacto", "nerfacto_trainer", "NerfactoTrainer")])
def test_gpu_training_reduces_loss(family, module, cls, tmp_path):
    import importlib

    mod = importlib.import_module(f"landmarksystem_b200.models.{family}.{module}")
    cfg = BaseConfig.from_file(os.path.join(ROOT, family, "confs", "synthetic_tiny.py"),
                               {"basedir": str(tmp_path), "device": "cuda", "n_iters": "300", "progress_refresh_rate": "1000",
                                "runtime": "Kernel"})
    trainer = getattr(mod, cls)(cfg)
    trainer.model.train()
    losses = []
    for trainer.iteration in range(300):
        losses.append(float(trainer.train_step(*trainer.data_mgr.get_rays(trainer.iteration))))
    assert np.mean(losses[-20:]) < 0.5 * np.mean(losses[:20]), (np.mean(losses[:20]), np.mean(losses[-20:]))


def test_volumetric_sampler_lean_output_matches_packed_samples():
    """The lean return (origins, directions, interval ends, validity) describes the same samples as the packed records."""
    from landmarksystem_b200.components.ray_samplers.volumetric_sampler import VolumetricSampler

    est = _grid(levels=1)
    o, d = _rays(32)
    rays = torch.cat((o, d, torch.arange(32.0)[:, None]), -1)
    sampler = VolumetricSampler(occupancy_grid=est, near_far=[0.1, 10.0], step_size=0.05, max_samples=64).eval()
    samples, valid = sampler(rays, training=False, render_stratified_sampling=False)
    o2, d2, ts, te, valid2 = sampler(rays, training=False, render_stratified_sampling=False, lean=True)
    assert torch.equal(valid, valid2) and torch.equal(samples.t_starts, ts) and torch.equal(samples.t_ends, te)
    z = 0.5 * (ts + te)
    xyz = o2[:, None] + d2[:, None] * z[..., None]
    assert torch.allclose(samples.data[..., 9:12][valid], xyz[valid]) and torch.allclose(samples.data[..., 6:9][valid], d2[:, None].expand_as(xyz)[valid])
    assert torch.equal(samples.data[:, 0, 4], rays[:, 6])


@pytest.mark.gpu
def test_ngp_kernel_glue_equals_tensor_op_glue(tmp_path):
    """One forward + backward of the Instant-NGP field with the per-sample glue as kernels and as tensor ops: same image,
    same gradients (both run the same fused heads, so only summation order differs)."""
    from landmarksystem_b200.models.instant_ngp.instant_ngp_trainer import NGPTrainer

    cfg = BaseConfig.from_file(os.path.join(ROOT, "instant_ngp", "confs", "synthetic_tiny.py"),
                               {"basedir": str(tmp_path), "device": "cuda", "n_iters": "1", "progress_refresh_rate": "1000",
                                "runtime": "Kernel"})
    trainer = NGPTrainer(cfg)
    model = trainer.model.train()
    rays, _ = trainer.data_mgr.get_rays(0)[:2]
    results = []
    for use_kernels in (True, False):
        model._kernel_glue = (lambda r, keep=model.__class__._kernel_glue: keep(model, r)) if use_kernels else (lambda r: False)
        torch.manual_seed(7)                                   # same stratified jitter in both passes
        table = next(model.mlp_base_grid.parameters())
        sink = getattr(table, "_lmb_grad_sink", None)          # the trainer gives the table a persistent accumulator
        for p in model.parameters():
            p.grad = None
        if sink is not None:
            sink.zero_()
        out = model(rays)["rgb_map"]
        out.square().sum().backward()
        table_grad = sink if sink is not None else table.grad
        results.append((out.detach().clone(), table_grad.detach().clone().float(),
                        model.embedding_appearance.weight.grad.detach().clone()))
    (img_k, g_k, e_k), (img_t, g_t, e_t) = results
    assert torch.allclose(img_k, img_t, atol=2e-3)
    assert torch.allclose(g_k, g_t, atol=2e-3 * float(g_t.abs().max()) + 1e-7)
    assert torch.allclose(e_k, e_t, atol=2e-2 * float(e_t.abs().max()) + 1e-7)


def test_ngp_restatement_baseline_trains():
    """The PyTorch restatement that serves as the Instant-NGP baseline runs end to end and reduces its loss (CPU, tiny)."""
    from baseline.ngp_restatement import Trainer

    torch.manual_seed(0)
    tr = Trainer([[-1, -1, -1], [1, 1, 1]], step=0.1, max_samples=24, device="cpu", grid_res=8, chunk_rays=64, levels=4,
                 features=2, log2_size=10, base_res=4, max_res=32, n_cameras=4, app_dim=8)
    R = 128
    ang = torch.rand(R) * 6.28
    o = torch.stack((3 * torch.cos(ang), 3 * torch.sin(ang), torch.rand(R) - 0.5), -1)
    rays = torch.cat((o, torch.nn.functional.normalize(torch.rand(R, 3) * 1.6 - 0.8 - o, dim=-1)), -1)
    target = torch.rand(R, 3) * 0.2 + 0.6
    losses = [tr.train_step(rays, target, torch.zeros(R)) for _ in range(25)]
    assert losses[-1] < 0.3 * losses[0]


def test_ngp_reuses_the_culling_pass_rows_for_the_survivors(tmp_path):
    """The step's forward takes hash features / head outputs of the sampler's density query for the samples that survived
    the culling: the row bookkeeping (survivor slot -> slot before the compaction -> row of the query), with the query
    covering all R x S slots and covering a subset."""
    from landmarksystem_b200.models.instant_ngp.instant_ngp_trainer import NGPTrainer

    cfg = BaseConfig.from_file(os.path.join(ROOT, "instant_ngp", "confs", "synthetic_tiny.py"),
                               {"basedir": str(tmp_path), "device": "cpu", "n_iters": "1", "datadir": "ring:3:12x12:14:3",
                                "batch_size": "64", "progress_refresh_rate": "100"})
    model = NGPTrainer(cfg).model.train()
    R, S = 5, 6
    g = torch.Generator().manual_seed(0)
    for subset in (False, True):
        marched = (torch.rand(R, S, generator=g) < 0.8) if subset else torch.ones(R, S, dtype=torch.bool)
        marched = marched.sort(dim=1, descending=True).values                 # marched samples fill a row's front
        queried = marched.reshape(-1).nonzero(as_tuple=True)[0]
        n = queried.numel()
        feat, h = torch.arange(n)[:, None].float().repeat(1, 4), torch.arange(n)[:, None].float().repeat(1, 2) + 0.5
        keep = marched & (torch.rand(R, S, generator=g) < 0.6)
        source = torch.zeros(R, S, dtype=torch.int32)
        for r in range(R):
            kept = keep[r].nonzero(as_tuple=True)[0]
            source[r, : kept.numel()] = kept.to(torch.int32)
        counts = keep.sum(1)
        survivors = (torch.arange(S)[None] < counts[:, None]).reshape(-1).nonzero(as_tuple=True)[0]
        model._cull_cache = {"feat": feat, "h": h}
        model.occupancy_grid.last_cull = {"queried": queried if subset else None, "source": source, "n_queried": n}
        got_feat, got_h = model._cached_field_rows(survivors, S)
        row_of_slot = torch.full((R * S,), -1, dtype=torch.long)
        row_of_slot[queried] = torch.arange(n)
        want = row_of_slot[keep.reshape(-1).nonzero(as_tuple=True)[0]]        # kept slots in row-major order = survivors' order
        assert torch.equal(got_feat[:, 0].long(), want) and torch.equal(got_h[:, 0], want.float() + 0.5)
        assert model._cull_cache is None                                       # consumed
    # nothing culled: the cached tensors are handed over as they are
    n = R * S
    feat, h = torch.zeros(n, 4), torch.zeros(n, 2)
    model._cull_cache = {"feat": feat, "h": h}
    model.occupancy_grid.last_cull = {"queried": None, "source": torch.arange(S, dtype=torch.int32).repeat(R, 1), "n_queried": n}
    got_feat, got_h = model._cached_field_rows(torch.arange(n), S)
    assert got_feat is feat and got_h is h

"""Model-parallel rendering by spatial blocks: per-block partial composites merged in entry order reproduce the
single-model render (CPU; the cross-GPU kernel version runs in tests/multigpu/worker_mp_render.py)."""
import torch

from landmarksystem_b200.components.scene import SceneManager
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF, GridNeRFConfig
from landmarksystem_b200.parallel.composite_merge import merge_reference
from landmarksystem_b200.parallel.mp_render import ModelParallelRenderer, slice_model_to_block_window
from landmarksystem_b200.utils import Config


def _build(division):
    mc = GridNeRFConfig(resMode=[1], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0, fea2denseAct="relu")
    cfg = Config(dict(mc))
    cfg.update(is_train=False, device=torch.device("cpu"), lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=division,
               branch_parallel=False, channel_parallel=False, DDP=False, sampling_opt=False)
    sm = SceneManager(cfg)
    torch.manual_seed(0)
    model = GridNeRF(sm.aabb, [32 * division[0], 32 * division[1], 16], cfg.device, near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    for p in model.density_encoding.parameters():
        p.data.abs_().mul_(3.0)
    return model.eval(), sm


def _rays(n=512):
    g = torch.Generator().manual_seed(5)
    o = torch.cat((torch.rand(n, 2, generator=g) * 3.6 - 1.8, torch.full((n, 1), 2.0)), -1)
    d = torch.nn.functional.normalize(torch.cat((torch.randn(n, 2, generator=g) * 0.8, -torch.ones(n, 1)), -1), dim=-1)
    return torch.cat((o, d, torch.zeros(n, 1)), -1)


def test_block_partials_merge_to_the_full_render():
    division = [2, 2]
    full, _ = _build(division)
    rays = _rays()
    parts = []
    for r in range(4):
        m, sm = _build(division)
        sm.assign_local_block_partition([1, 1])
        sm.assign_relative_block_idx(r)
        for enc in (m.density_encoding, m.rgb_encoding):
            for plist in (enc.plane_coef, enc.line_coef):
                for p in plist:
                    p.data = p.data[r:r + 1].contiguous()
        parts.append(m.render_partial(rays, 64))
    # the same through the engine's helper: two ranks, one band of block rows each
    banded = []
    for r in range(2):
        m, _ = _build(division)
        assert slice_model_to_block_window(m, r, 2) == (2 * r, 2)
        assert m.density_encoding.plane_coef[0].shape[0] == 2
        banded.append(m.render_partial(rays, 64))
    out2 = merge_reference(torch.stack(banded), bg=1.0 if full.renderer.white_bg else 0.0)
    out = merge_reference(torch.stack(parts), bg=1.0 if full.renderer.white_bg else 0.0)
    with torch.no_grad():
        ref_rgb, ref_depth = full(rays, N_samples=64)
    assert float(out[:, 5].max()) > 0.2
    assert torch.allclose(out[:, :3].clamp(0, 1), ref_rgb, atol=1e-5)
    assert torch.allclose(out[:, 4], ref_depth, atol=1e-5)
    assert torch.allclose(out2[:, :3].clamp(0, 1), ref_rgb, atol=1e-5) and torch.allclose(out2[:, 4], ref_depth, atol=1e-5)


def test_single_rank_renderer_equals_model():
    full, _ = _build([1, 1])
    rays = _rays(256)
    rgb, depth, acc = ModelParallelRenderer(full, 256).render(rays, N_samples=64, chunk=100)
    with torch.no_grad():
        ref_rgb, ref_depth = full(rays, N_samples=64)
    assert torch.allclose(rgb, ref_rgb, atol=1e-5) and torch.allclose(depth, ref_depth, atol=1e-5)

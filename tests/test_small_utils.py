"""Small utilities that the larger tests only touch indirectly: ray / box filtering, graphics helpers, SH colour
conversion, RAdam rectification against ``torch.optim.RAdam``, RNG snapshots, iterators and offload bookkeeping."""
import math
import os
import random

import numpy as np
import pytest
import torch


def test_ray_box_filter_and_graphics_helpers():
    from landmarksystem_b200.components.data.datasets.ray_utils import filtering_rays
    from landmarksystem_b200.components.utils.graphics_utils import (focal2fov, fov2focal, geom_transform_points,
                                                                     getProjectionMatrix, getWorld2View, getWorld2View2)

    aabb = torch.tensor([[-1.0, -1.0, -1.0], [1.0, 1.0, 1.0]])
    rays = torch.tensor([[0.0, 0.0, 5.0, 0.0, 0.0, -1.0],          # straight down into the box
                         [3.0, 0.0, 5.0, 0.0, 0.0, -1.0],          # parallel, beside the box
                         [0.0, 0.0, 5.0, 1.0, 0.0, 0.0],           # above the box, flying sideways
                         [-5.0, 0.2, 0.3, 1.0, 0.0, 0.0]])         # through the box along x
    assert filtering_rays(aabb, rays, chunk=3).tolist() == [True, False, False, True]
    assert math.isclose(focal2fov(fov2focal(0.9, 640), 640), 0.9) and math.isclose(fov2focal(math.pi / 2, 100), 50.0)
    R, t = np.eye(3, dtype=np.float32), np.array([1.0, 2.0, 3.0], dtype=np.float32)
    assert np.allclose(getWorld2View(R, t), getWorld2View2(R, t))
    shifted = getWorld2View2(R, t, translate=np.array([1.0, 0.0, 0.0]), scale=2.0)
    centre = np.linalg.inv(shifted)[:3, 3]
    assert np.allclose(centre, (np.array([-1.0, -2.0, -3.0]) + [1.0, 0.0, 0.0]) * 2.0, atol=1e-6)
    proj = getProjectionMatrix(0.1, 100.0, 0.8, 0.6).transpose(0, 1)
    pts = torch.tensor([[0.0, 0.0, 1.0], [0.3, -0.2, 5.0]])
    ndc = geom_transform_points(pts, proj)
    assert torch.allclose(ndc[0, :2], torch.zeros(2), atol=1e-6)            # a point on the axis projects to the centre
    assert math.isclose(float(ndc[1, 0]), 0.3 / (5.0 * math.tan(0.4)), rel_tol=1e-5)


def test_sh_colour_round_trip_and_l2():
    from landmarksystem_b200.components.utils.loss_utils import l1_loss, l2_loss
    from landmarksystem_b200.components.utils.sh_utils import RGB2SH, SH2RGB, eval_sh

    rgb = torch.rand(7, 3)
    assert torch.allclose(SH2RGB(RGB2SH(rgb)), rgb, atol=1e-6)
    dc = RGB2SH(rgb)[:, :, None]                                            # degree 0: colour independent of direction
    assert torch.allclose(eval_sh(0, dc, torch.randn(7, 3)) + 0.5, rgb, atol=1e-6)
    a, b = torch.tensor([1.0, 2.0, 4.0]), torch.tensor([1.0, 0.0, 1.0])
    assert float(l2_loss(a, b)) == pytest.approx((0 + 4 + 9) / 3) and float(l1_loss(a, b)) == pytest.approx(5 / 3)


def test_radam_step_size_matches_torch():
    from landmarksystem_b200.ops.optim import radam_step_size

    lr, b1, b2, eps = 1e-2, 0.9, 0.999, 1e-15
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(5))
    ref = torch.optim.RAdam([p], lr=lr, betas=(b1, b2), eps=eps)
    m, v, mine = torch.zeros(5), torch.zeros(5), p.detach().clone()
    for step in range(1, 13):                                              # crosses the step where rectification turns on
        g = torch.randn(5)
        p.grad = g.clone()
        ref.step()
        m, v = b1 * m + (1 - b1) * g, b2 * v + (1 - b2) * g * g
        size, adaptive = radam_step_size(lr, b1, b2, step)
        mine = mine - size * (m / (v.sqrt() + eps) if adaptive else m)
        assert torch.allclose(mine, p.detach(), atol=1e-6), step
    assert radam_step_size(lr, b1, b2, 1)[1] is False and radam_step_size(lr, b1, b2, 12)[1] is True


def test_rng_snapshot_restores_all_generators():
    from landmarksystem_b200.runtime import checkpoint as ck

    state = ck.capture_rng_state()
    first = (torch.rand(3), np.random.rand(3), random.random())
    ck.restore_rng_state(state)
    again = (torch.rand(3), np.random.rand(3), random.random())
    assert torch.equal(first[0], again[0]) and np.array_equal(first[1], again[1]) and first[2] == again[2]


def test_iterators_key_cleaning_and_offload_bookkeeping(tmp_path):
    from types import SimpleNamespace

    from landmarksystem_b200.components.utils.system_utils import mkdir_p, searchForMaxIteration
    from landmarksystem_b200.render.offload.utils import (assign_block_to_pose, list_key_for_block,
                                                          search_maximum_memory_used_per_param)
    from landmarksystem_b200.train.utils import CircularIterator, rm_redundant_words_in_state_dict

    it = CircularIterator([1, 2, 3])
    assert [next(it) for _ in range(7)] == [1, 2, 3, 1, 2, 3, 1]
    cleaned = rm_redundant_words_in_state_dict({"module.a.module.w": 1, "b": 2}, ["module."])
    assert cleaned == {"a.w": 1, "b": 2}
    for n in (7, 300, 25):
        mkdir_p(str(tmp_path / "point_cloud" / f"iteration_{n}"))
    assert searchForMaxIteration(str(tmp_path / "point_cloud")) == 300

    aabb = torch.tensor([[-2.0, -4.0, 0.0], [2.0, 4.0, 1.0]])
    pose = torch.eye(4)
    pose[:3, 3] = torch.tensor([1.5, -3.9, 7.0])
    assert assign_block_to_pose(pose, aabb, [2, 4]) == 1 * 4 + 0
    assert assign_block_to_pose(torch.tensor([-9.0, 9.0, 0.0]), aabb, [2, 4]) == 0 * 4 + 3      # clamped to the border
    assert list_key_for_block("grid.tcnn_encoding.2.params", 2) == "grid.tcnn_encoding.{}.params"
    assert list_key_for_block("grid.tcnn_encoding.2.params", 1) is None and list_key_for_block("mlp.weight", 0) is None
    blocks = [SimpleNamespace(state_dict={"p": torch.zeros(10 * (b + 1))}) for b in range(4)]   # uneven 2x2 blocks
    assert search_maximum_memory_used_per_param(blocks, [2, 2], [1, 2])["p"] == 30 + 40        # the largest 1x2 window

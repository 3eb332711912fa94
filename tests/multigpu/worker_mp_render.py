"""Worker (>= 2 GPUs): model-parallel rendering.  Every rank holds one spatial block of a GridNeRF scene, renders
its own ray segments and the cross-GPU ordered composite kernel merges them; the result is compared with the
single-model render of the whole scene."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from landmarksystem_b200.components.scene import SceneManager  # noqa: E402
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF, GridNeRFConfig  # noqa: E402
from landmarksystem_b200.parallel.mp_render import ModelParallelRenderer  # noqa: E402
from landmarksystem_b200.utils import Config  # noqa: E402


def build(division, window=None, origin=0):
    mc = GridNeRFConfig(resMode=[1], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0, fea2denseAct="relu")
    cfg = Config(dict(mc))
    cfg.update(is_train=False, device=torch.device("cuda", torch.cuda.current_device()), lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5],
               plane_division=division, branch_parallel=False, channel_parallel=False, DDP=False, sampling_opt=False)
    if window is not None:
        cfg.update(local_block_partition=window, relative_block_idx=origin)
    sm = SceneManager(cfg)
    torch.manual_seed(0)
    n_blocks = division[0] * division[1]
    model = GridNeRF(sm.aabb, [32 * division[0], 32 * division[1], 16], cfg.device, near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    for p in model.density_encoding.parameters():
        p.data.abs_().mul_(3.0)
    assert model.density_encoding.plane_coef[0].shape[0] == n_blocks
    return model.eval(), sm


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    division = [world, 1]
    full, _ = build(division)
    # this rank's model: same weights, only block `rank` resident
    mine, sm = build(division)
    sm.assign_local_block_partition([1, 1])
    sm.assign_relative_block_idx(rank)
    for enc in (mine.density_encoding, mine.rgb_encoding):
        for plist in (enc.plane_coef, enc.line_coef):
            for p in plist:
                p.data = p.data[rank:rank + 1].contiguous()
    g = torch.Generator().manual_seed(5)
    n = 4096
    o = torch.cat((torch.rand(n, 2, generator=g) * 3.6 - 1.8, torch.full((n, 1), 2.0)), -1)
    d = torch.nn.functional.normalize(torch.cat((torch.randn(n, 2, generator=g) * 0.8, -torch.ones(n, 1)), -1), dim=-1)
    rays = torch.cat((o, d, torch.zeros(n, 1)), -1).cuda()
    renderer = ModelParallelRenderer(mine, n)
    rgb, depth, acc = renderer.render(rays, N_samples=64)
    renderer.merger.barrier.check()
    with torch.no_grad():
        ref_rgb, ref_depth = full(rays, N_samples=64)
    err = float((rgb - ref_rgb).abs().max())
    derr = float((depth - ref_depth).abs().max())
    assert err < 2e-3 and derr < 2e-2, (err, derr)
    assert float(acc.max()) > 0.2                     # the scene is not empty
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(); torch.cuda.synchronize()
    s.record()
    for _ in range(5):
        renderer.render(rays, N_samples=64)
    e.record(); torch.cuda.synchronize()
    if rank == 0:
        print("MP_RENDER_RESULTS " + json.dumps({"world": world, "max_rgb_err": err, "max_depth_err": derr,
              "ms_per_4096_rays": s.elapsed_time(e) / 5}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

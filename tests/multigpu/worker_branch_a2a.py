"""Worker (>= 2 GPUs): branch-parallel GridNeRF where every rank brings its own rays and samples are
dispatched to the owning GPU over peer memory, checked against the replicate-and-all-reduce mode."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from landmarksystem_b200.comm.train_groups import init_train_groups  # noqa: E402
from landmarksystem_b200.components.scene import SceneManager  # noqa: E402
from landmarksystem_b200.convertor import ComponentConvertorFactory  # noqa: E402
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF, GridNeRFConfig  # noqa: E402
from landmarksystem_b200.utils import Config  # noqa: E402


def build(division, mode):
    mc = GridNeRFConfig(resMode=[1, 2], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0, branch_dispatch=mode)
    cfg = Config(dict(mc))
    cfg.update(is_train=True, device=torch.device("cuda", torch.cuda.current_device()), lb=[-2.0, -2.0, -0.5],
               ub=[2.0, 2.0, 0.5], plane_division=division, branch_parallel=True, channel_parallel=False,
               model_parallel_and_DDP=False, DDP=False)
    init_train_groups(cfg)
    sm = SceneManager(cfg)
    torch.manual_seed(0)
    model = GridNeRF(sm.aabb, [32 * division[0], 32 * division[1], 16], cfg.device, near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    model = ComponentConvertorFactory.get_convertor("parallelize").convert(model, cfg)
    for mod in (model.feature2density, model.rgb_decoder):
        for p in mod.parameters():
            dist.broadcast(p.data, src=0)
    for p in model.density_encoding.parameters():
        p.data.abs_().mul_(2.0)
    return model.eval(), cfg      # eval(): no jitter-free difference, no random white background


def rays_for(rank, n=2048):
    g = torch.Generator().manual_seed(100 + rank)
    o = torch.cat((torch.rand(n, 2, generator=g) * 3.6 - 1.8, torch.full((n, 1), 3.0)), -1)
    d = torch.nn.functional.normalize(torch.cat((torch.randn(n, 2, generator=g) * 0.3, -torch.ones(n, 1)), -1), dim=-1)
    return torch.cat((o, d, torch.zeros(n, 1)), -1).cuda()


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    division = {2: [2, 1], 4: [2, 2], 8: [2, 4]}[world]
    ref_model, _ = build(division, "allreduce")
    a2a_model, _ = build(division, "a2a")
    a2a_model.load_state_dict(ref_model.state_dict())
    target = torch.rand(2048, 3, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))

    def sample_free(model, rays):
        torch.manual_seed(1234)          # same jitter in both modes
        return model(rays, N_samples=48)["rgb_map"]

    # a2a: each rank its own rays
    mine = rays_for(rank)
    out_a = sample_free(a2a_model, mine)
    (((out_a - target) ** 2).mean()).backward()
    # reference mode: all ranks evaluate every rank's rays in turn
    out_r = None
    for r in range(world):
        o = sample_free(ref_model, rays_for(r))
        (((o - target) ** 2).mean()).backward()
        if r == rank:
            out_r = o.detach()
    err = (out_a.detach() - out_r).abs().max().item()
    assert err < 1e-4, err
    gerr = 0.0
    for (n1, p1), (n2, p2) in zip(a2a_model.named_parameters(), ref_model.named_parameters()):
        if "encoding" not in n1:
            continue                       # replicated heads hold partial sums until the MP gradient sync
        g1, g2 = p1.grad, p2.grad
        assert g1 is not None and g2 is not None, n1
        scale = g2.abs().max().item() + 1e-12
        gerr = max(gerr, (g1 - g2).abs().max().item() / scale)
    assert gerr < 1e-3, gerr
    a2a_model._a2a.check()

    # the same exchange with the kernel path on the owner (tcgen05 colour head forward + backward, device-side
    # row counts end to end: no host synchronisation inside the step), against the replicated PyTorch heads
    fused_model, fcfg = build(division, "a2a")
    fused_model.load_state_dict(ref_model.state_dict())
    fcfg.fused_mlp_train = True
    fused_model.rgb_decoder.use_fused = True
    assert fused_model._fused_app_stage_ok(mine)
    for p in ref_model.parameters():
        p.grad = None
    out_f = sample_free(fused_model, mine)
    (((out_f - target) ** 2).mean()).backward()
    for r in range(world):
        (((sample_free(ref_model, rays_for(r)) - target) ** 2).mean()).backward()
    ferr = (out_f.detach() - out_r).abs().max().item()
    assert ferr < 3e-2, ferr
    fgerr = 0.0
    for (n1, p1), (n2, p2) in zip(fused_model.named_parameters(), ref_model.named_parameters()):
        if "encoding" not in n1:
            continue
        fgerr = max(fgerr, float((p1.grad - p2.grad).norm() / (p2.grad.norm() + 1e-12)))
    assert fgerr < 0.15, fgerr
    fused_model.rgb_decoder._lmb_packed.check_status()
    fused_model._a2a.check()
    assert int(fused_model._a2a.overflow.item()) == 0

    # timing of a training-shaped forward+backward with 8192 rays x 128 samples per rank
    big = rays_for(rank, 8192)
    tgt = torch.rand(8192, 3, device="cuda")

    def step(model, rays):
        out = model(rays, N_samples=128)["rgb_map"]
        ((out - tgt) ** 2).mean().backward()

    def timed(fn, iters=5):
        for _ in range(2):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record(); torch.cuda.synchronize()
        ms = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    ms_a2a = timed(lambda: step(a2a_model, big))
    ms_fused = timed(lambda: step(fused_model, big))
    allrays = torch.cat([rays_for(r, 8192) for r in range(world)])
    tgt_all = torch.rand(8192 * world, 3, device="cuda")

    def step_ref():
        out = ref_model(allrays, N_samples=128)["rgb_map"]
        ((out - tgt_all) ** 2).mean().backward()

    ms_ref = timed(step_ref, iters=3)
    if rank == 0:
        print("BRANCH_A2A_RESULTS " + json.dumps({"world": world, "max_err": err, "grad_rel_err": gerr,
              "a2a_ms_per_step": ms_a2a, "a2a_kernel_path_ms_per_step": ms_fused, "kernel_path_max_err": ferr,
              "kernel_path_grad_rel_err": fgerr, "replicate_allreduce_ms_per_step": ms_ref,
              "rays_per_step": 8192 * world}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

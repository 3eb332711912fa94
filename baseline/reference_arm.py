"""Reference arm of the benchmark.

Runs the reference's own GridNeRF trainer (``benchmarks/nerf/gridnerf/gridnerf_trainer.py`` copied
unmodified into ``baseline/_ref``) on the benchmark configuration and prints the same JSON line as
``bench.py``'s own arm.  None of this framework's models, kernels or engine is imported here.

What the harness adds around the reference code, without touching it:
* stand-ins for third-party packages that are not installed offline and that the benchmarked code
  path never calls (``lpips``, ``imageio``, ``kornia.create_meshgrid``, ``plyfile``, ...), plus
  ``torch_efficient_distloss.eff_distloss`` restated in PyTorch (the reference evaluates it every
  step for its returned dict);
* a tiny MatrixCity-format dataset written to a temp dir so the reference ``DatasetManager`` builds
  through its own loader;
* the benchmark grid size is reached through the model's own ``upsample_volume_grid`` followed by
  the trainer's ``create_optimizer`` (what its schedule does after an upsample);
* ``data_mgr.get_rays`` is wrapped to feed the shared synthetic ray pool (pinned host -> device
  every call) and to bracket the timed iterations of the stock ``train()`` loop with CUDA events.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import types


class _StopBench(Exception):
    pass


def _install_shims():
    import numpy as np
    import torch

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    def eff_distloss(w, m, interval):
        loss_uni = (1 / 3) * (interval * w.pow(2)).sum(dim=-1).mean()
        wm = w * m
        w_cum, wm_cum = w.cumsum(dim=-1), wm.cumsum(dim=-1)
        loss_bi = 2 * (wm[..., 1:] * w_cum[..., :-1] - w[..., 1:] * wm_cum[..., :-1]).sum(dim=-1).mean()
        return loss_bi + loss_uni

    def create_meshgrid(height, width, normalized_coordinates=True, device=None, dtype=torch.float32):
        xs = torch.linspace(0, width - 1, width, device=device, dtype=dtype)
        ys = torch.linspace(0, height - 1, height, device=device, dtype=dtype)
        if normalized_coordinates:
            xs, ys = (xs / (width - 1) - 0.5) * 2, (ys / (height - 1) - 0.5) * 2
        grid = torch.stack(torch.meshgrid(xs, ys, indexing="ij"), dim=-1)
        return grid.permute(1, 0, 2).unsqueeze(0)

    def imwrite(path, arr, *a, **k):
        from PIL import Image

        Image.fromarray(np.asarray(arr)).save(path)

    class _Unavailable:
        def __init__(self, *a, **k):
            raise RuntimeError("this third-party package is not installed offline")

    if "torch_efficient_distloss" not in sys.modules:
        mod("torch_efficient_distloss", eff_distloss=eff_distloss)
    for name, attrs in (("kornia", dict(create_meshgrid=create_meshgrid)),
                        ("imageio", dict(imwrite=imwrite, imread=lambda p: np.asarray(__import__("PIL.Image").Image.open(p)))),
                        ("lpips", dict(LPIPS=_Unavailable)),
                        ("plyfile", dict(PlyData=_Unavailable, PlyElement=_Unavailable)),
                        ("laspy", {}), ("torch_scatter", dict(scatter_max=_Unavailable)),
                        ("colorama", dict(Fore=types.SimpleNamespace(RED="", GREEN="", YELLOW="", RESET=""),
                                          Style=types.SimpleNamespace(RESET_ALL=""))),
                        ("opt_gaussian_rasterization", dict(GaussianRasterizationSettings=_Unavailable,
                                                            GaussianRasterizer=_Unavailable)),
                        ("nerfacc", dict(OccGridEstimator=_Unavailable))):
        try:
            __import__(name)
        except Exception:
            mod(name, **attrs)
    try:
        import wandb  # noqa: F401
    except Exception:
        mod("wandb", init=lambda *a, **k: None, config=types.SimpleNamespace(update=lambda *a, **k: None))


def _write_dataset(root, lb, ub):
    """Two 32x18 training images and one test image in MatrixCity layout."""
    import numpy as np
    from PIL import Image

    os.makedirs(os.path.join(root, "train"), exist_ok=True)
    os.makedirs(os.path.join(root, "test"), exist_ok=True)
    cx, cy = (lb[0] + ub[0]) / 2, (lb[1] + ub[1]) / 2
    for split, n in (("train", 2), ("test", 1)):
        frames = []
        for k in range(n):
            name = f"{split}/{k:04d}.png"
            Image.fromarray((np.random.rand(18, 32, 3) * 255).astype(np.uint8)).save(os.path.join(root, name))
            c2w = np.eye(4)
            c2w[:3, 3] = [cx + 10 * k, cy, lb[2] + 400.0]   # nadir camera (looks along -z)
            frames.append({"file_path": name, "transform_matrix": c2w.tolist()})
        with open(os.path.join(root, f"transforms_{split}.json"), "w", encoding="utf-8") as fh:
            json.dump({"fl_x": 27.7, "w": 32, "h": 18, "frames": frames}, fh)


_CONF = '''
from landmark.nerf_components.configs import DatasetConfig, TrainConfig
from benchmarks.nerf.gridnerf.gridnerf import GridNeRFConfig
train_config = TrainConfig(model_name="GridNeRF", expname="gridnerf_ref_bench", basedir={basedir!r}, n_iters={n_iters},
    batch_size={batch}, progress_refresh_rate=1000000, vis_every=100000000, N_vis=0, random_seed=0,
    branch_parallel={branch}, plane_division={division}, print_timestamp=False)
dataset_config = DatasetConfig(dataset_name="matrixcity", datadir={datadir!r}, lb={lb}, ub={ub}, downsample_train=1)
model_config = GridNeRFConfig(resMode=[1], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True,
    fea2denseAct="relu", view_pe=2, fea_pe=2, featureC=128, N_voxel_init=64**3, N_voxel_final=64**3, upsamp_list=[],
    update_AlphaMask_list=[], nSamples=128, step_ratio=10.0, train_near_far=[10.0, 2000.0], lr_init=0.02,
    lr_basis=1e-3, distance_scale=25, appearance_embedding_size=2, L1_weight_inital=0.0, L1_weight_rest=0.0)
config = [train_config, dataset_config, model_config]
'''


def run_reference(args, DIVISIONS, RAYS_PER_GPU, SAMPLES, BLOCK_M, PLANE, LINE, make_ray_pool, ClockSampler):
    ref_root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    if not os.path.isdir(os.path.join(ref_root, "landmark")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not hold the reference tree"}))
        return
    try:
        _run(args, ref_root, DIVISIONS, RAYS_PER_GPU, SAMPLES, BLOCK_M, PLANE, LINE, make_ray_pool, ClockSampler)
    except _StopBench:
        raise
    except Exception as exc:  # report, do not crash the driver
        if int(os.environ.get("RANK", 0)) == 0:
            msg = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:300]
            print(json.dumps({"impl": "reference", "unavailable": f"reference trainer failed here: {msg}"}), flush=True)


def _run(args, ref_root, DIVISIONS, RAYS_PER_GPU, SAMPLES, BLOCK_M, PLANE, LINE, make_ray_pool, ClockSampler):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ref_root)
    _install_shims()
    n = args.gpus
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    assert world == n
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    nx, ny = DIVISIONS[n]
    lb, ub = [0.0, 0.0, 0.0], [BLOCK_M[0] * nx, BLOCK_M[1] * ny, BLOCK_M[2]]
    steps, warmup = args.steps, args.warmup
    global_batch = RAYS_PER_GPU * n
    work = os.path.join(tempfile.gettempdir(), f"lmb_ref_bench_{n}")
    if rank == 0:
        _write_dataset(os.path.join(work, "data"), lb, ub)
    conf_path = os.path.join(work, f"conf_rank{rank}.py")
    os.makedirs(work, exist_ok=True)
    with open(conf_path, "w", encoding="utf-8") as fh:
        fh.write(_CONF.format(basedir=os.path.join(work, "log"), n_iters=warmup + steps + 1, batch=global_batch,
                              branch=(n > 1), division=[nx, ny], datadir=os.path.join(work, "data"), lb=lb, ub=ub))

    from benchmarks.nerf.gridnerf.gridnerf_trainer import GridNeRFTrainer
    from landmark.nerf_components.configs import BaseConfig

    if world > 1 and rank != 0:
        import time
        time.sleep(3)  # let rank 0 write the dataset before the loaders open it
    cfg = BaseConfig.from_file(conf_path)
    trainer = GridNeRFTrainer(cfg)
    # bring the grids to the benchmark resolution through the model's own API, then a fresh optimiser
    trainer.module.upsample_volume_grid([PLANE * nx, PLANE * ny, LINE])
    trainer.optimizer = trainer.create_optimizer()
    dev = cfg.device

    pool_steps = min(steps + warmup + 1, 16)
    rays, rgbs, idxs = make_ray_pool(global_batch * pool_steps, lb, ub, seed=1234)
    idxs = idxs % 2
    host = torch.cat((rays, rgbs, idxs[:, None]), -1).view(pool_steps, global_batch, 10).pin_memory()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(torch.cuda.current_device())
    state = {"k": 0}

    def get_rays(iteration):
        k = state["k"]
        if k == warmup:
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            if rank == 0:
                sampler.start()
            start.record()
        if k == warmup + steps:
            end.record()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            raise _StopBench()
        state["k"] = k + 1
        b = host[k % pool_steps].to(dev, non_blocking=True)
        return b[:, :6], b[:, 6:9], b[:, 9]

    trainer.data_mgr.get_rays = get_rays
    try:
        trainer.train()
    except _StopBench:
        pass
    ms = torch.tensor([start.elapsed_time(end)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        value = global_batch * steps / (ms / 1e3)
        print(json.dumps({
            "metric": "train rays/s", "value": value, "unit": "rays/s", "n_gpus": n, "steps": steps, "warmup": warmup,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16 autocast (reference default)", "data": "synthetic", "impl": "reference",
            "config": {"model": "GridNeRF branch-parallel large scene", "global_batch": global_batch,
                       "seq_len": SAMPLES, "parallelism": f"branch{nx}x{ny}" if n > 1 else "single",
                       "planes": f"{PLANE}^2 x (16+48)ch fp32 per GPU", "lines": LINE,
                       "l2_policy": "inputs larger than L2"},
            "clocks": clocks,
            "e2e": {"value": value, "unit": "rays/s", "ms_per_step": ms / steps,
                    "h2d_bytes_per_step": global_batch * 10 * 4, "d2h_bytes_per_step": 4},
            "gpu_launches": 0,
        }), flush=True)
    if dist.is_initialized():
        if world > 1:
            dist.barrier()
        dist.destroy_process_group()           # the reference initialises a group even for one rank

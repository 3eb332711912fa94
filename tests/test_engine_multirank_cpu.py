"""The rendering engine on several CPU ranks (gloo): data parallel, channel ("tensor") parallel and both together give
rank 0 the image one process renders - the reference's multi-device render tests
(tests/test_inference_framework/test_multi_device/test_torch_parallel_inference.py:22-313) without GPUs."""
import multiprocessing as mp
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gridnerf_config(folder, **extra):
    from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRFConfig
    from landmarksystem_b200.utils import Config

    mc = GridNeRFConfig(resMode=[1, 2], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0, n_importance=48, sampling_opt=True)
    cfg = Config(dict(mc))
    cfg.update(is_train=False, device="cpu", lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=[1, 1],
               branch_parallel=False, ckpt=os.path.join(folder, "state_dict.th"), kwargs=os.path.join(folder, "kwargs.th"))
    cfg.update(extra)
    return cfg


def _ngp_config(folder, **extra):
    from landmarksystem_b200.models.instant_ngp.instant_ngp import InstantNGPConfig
    from landmarksystem_b200.utils import Config

    mc = InstantNGPConfig(num_levels=4, base_res=8, max_res=64, log2_hashmap_size=12, grid_resolution=16, grid_levels=1,
                          train_near_far=[0.5, 6.0], appearance_embedding_size=4, render_step_size=0.05, cone_angle=0.0,
                          max_samples_per_ray=96, background_color="black", runtime="Torch",
                          render_stratified_sampling=False)
    cfg = Config(dict(mc))
    cfg.update(is_train=False, device="cpu", lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=[1, 1],
               branch_parallel=False, ckpt=os.path.join(folder, "state_dict.th"), kwargs=os.path.join(folder, "kwargs.th"),
               aabb_norm_range=[0, 1], **extra)
    return cfg


def _pose():
    from landmarksystem_b200.synthetic import look_at

    return look_at(torch.tensor([-0.9, 0.8, 3.0]), torch.tensor([-0.85, 0.8, 0.0]), up=(0.0, 1.0, 0.0))


def _save_models(folder):
    from landmarksystem_b200.components.scene import SceneManager
    from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF
    from landmarksystem_b200.models.instant_ngp.instant_ngp import InstantNGP

    torch.manual_seed(0)
    os.makedirs(os.path.join(folder, "grid"))
    os.makedirs(os.path.join(folder, "ngp"))
    cfg = _gridnerf_config(os.path.join(folder, "grid"))
    sm = SceneManager(cfg)
    grid = GridNeRF(sm.aabb, [32, 32, 16], "cpu", near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    for p in grid.density_encoding.parameters():
        p.data.abs_().mul_(3.0)
    grid.save_model(os.path.join(folder, "grid"))
    os.makedirs(os.path.join(folder, "grid22"))
    cfg = _gridnerf_config(os.path.join(folder, "grid22"), plane_division=[2, 2])
    sm = SceneManager(cfg)
    blocks = GridNeRF(sm.aabb, [64, 64, 16], "cpu", near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    for p in blocks.density_encoding.parameters():
        p.data.abs_().mul_(3.0)
    blocks.save_model(os.path.join(folder, "grid22"))
    cfg = _ngp_config(os.path.join(folder, "ngp"))
    sm = SceneManager(cfg)
    ngp = InstantNGP(sm.aabb, "cpu", [0.5, 6.0], scene_manager=sm, config=cfg)
    for p in ngp.mlp_base_grid.parameters():
        p.data.normal_(0, 1.0)
    ngp.save_model(os.path.join(folder, "ngp"))


def _render(kind, folder, parallel):
    import landmarksystem_b200 as lm
    from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF
    from landmarksystem_b200.models.instant_ngp.instant_ngp import InstantNGP
    from landmarksystem_b200.render.adapters import make_adapter
    from landmarksystem_b200.utils import Config

    if kind == "grid":
        cls, cfg = GridNeRF, _gridnerf_config(os.path.join(folder, "grid"))
    elif kind == "grid22":
        cls, cfg = GridNeRF, _gridnerf_config(os.path.join(folder, "grid22"), plane_division=[2, 2])
    else:
        cls, cfg = InstantNGP, _ngp_config(os.path.join(folder, "ngp"))
    inference = Config(runtime="Torch", kernel_fusion=False)
    parallel = dict(parallel) if parallel is not None else None
    offload = parallel.pop("offload", None) if parallel else None
    if parallel:
        inference.parallel_config = Config(parallel)
    if offload is not None:
        inference.offload_config = Config(offload)
    engine = lm.init_inference(cls, make_adapter(cls), cfg, inference)
    rank = int(os.environ.get("RANK", 0))
    out = engine(_pose(), 4096, 18, 24, 30.0) if rank == 0 else engine()
    return out[0].clone() if rank == 0 else None


def _worker(rank, world, port, folder, kind, parallel, queue):
    import traceback

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    try:
        image = _render(kind, folder, parallel)
        queue.put((rank, None, None if image is None else image.numpy()))
    except Exception:
        queue.put((rank, traceback.format_exc(), None))


def _run(world, folder, kind, parallel):
    ctx = mp.get_context("spawn")
    queue = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, folder, kind, parallel, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get() for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    for r in results:
        assert r[1] is None, r[1]
    return torch.from_numpy([r for r in results if r[0] == 0][0][2])


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("engine_models"))
    _save_models(folder)
    return folder


@pytest.mark.parametrize("kind,world,parallel", [
    ("grid", 2, {"tp_size": 1}),                     # data parallel: the rays of the frame dealt over two ranks
    ("grid", 2, {"tp_size": 2}),                     # channel parallel: every rank holds half of the feature channels
    ("grid", 4, {"tp_size": 2}),                     # two channel-parallel groups, data parallel across them
    ("ngp", 2, {"tp_size": 1}),
    ("grid22", 2, {"tp_size": 2}),                   # a block-stacked (branch-parallel) checkpoint rendered channel parallel
    # dynamic loading together with data parallelism: the ranks share the host reads of a new window (`use_nccl`)
    ("grid22", 2, {"tp_size": 1, "offload": {"local_plane_split": [2, 1], "plane_split": [2, 2], "use_nccl": True}}),
])
def test_engine_on_cpu_ranks_equals_one_process(models, kind, world, parallel):
    # a window shows only its own blocks, so the one-process image of that case is rendered through the same window
    alone = {"offload": dict(parallel["offload"], use_nccl=False)} if "offload" in parallel else None
    single = _render(kind, models, alone)
    assert single.shape == (18, 24, 4) and single[..., :3].float().std() > 1.0
    multi = _run(world, models, kind, parallel)
    assert (multi.float() - single.float()).abs().max() <= 1.0          # 8-bit rounding of sums taken in another order


def _evaluate(conf, over, ckpt):
    from landmarksystem_b200.configs import BaseConfig
    from landmarksystem_b200.models.instant_ngp.instant_ngp_evaluator import NGPEvaluator

    cfg = BaseConfig.from_file(conf, dict(over))
    cfg.is_train = False
    cfg.ckpt = ckpt
    cfg.render_stratified_sampling = False          # jitter-free renders: the split and the whole frame see the same samples
    return NGPEvaluator(cfg).eval()


def _eval_worker(rank, world, port, conf, over, ckpt, queue):
    import traceback

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    try:
        queue.put((rank, None, _evaluate(conf, over, ckpt)))
    except Exception:
        queue.put((rank, traceback.format_exc(), None))


def test_evaluator_splits_the_pixels_over_cpu_ranks(tmp_path):
    """The evaluator under two ranks (every rank renders half of each test image, reference:
    benchmarks/nerf/instant_ngp/instant_ngp_evaluator.py with a `*_ddp_render` configuration) reports the PSNR of one."""
    from landmarksystem_b200.configs import BaseConfig
    from landmarksystem_b200.models.instant_ngp.instant_ngp_trainer import NGPTrainer

    conf = os.path.join(ROOT, "landmarksystem_b200", "models", "instant_ngp", "confs", "synthetic_tiny.py")
    over = {"basedir": str(tmp_path), "device": "cpu", "n_iters": "3", "datadir": "ring:3:12x12:14:3", "batch_size": "64",
            "progress_refresh_rate": "100", "N_vis": "-1"}
    trainer = NGPTrainer(BaseConfig.from_file(conf, dict(over)))
    trainer.train()
    ckpt = os.path.join(trainer.logfolder, "state_dict.th")
    alone = _evaluate(conf, over, ckpt)
    ctx = mp.get_context("spawn")
    queue = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_eval_worker, args=(r, 2, port, conf, over, ckpt, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get() for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
    for r in results:
        assert r[1] is None, r[1]
    for r in results:
        assert abs(r[2] - alone) < 1e-3, (r[2], alone)


def _train_worker(rank, world, port, family, over, mode, queue):
    import importlib
    import traceback

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    try:
        from landmarksystem_b200.configs import BaseConfig

        name = "instant_ngp_trainer" if family == "instant_ngp" else "nerfacto_trainer"
        mod = importlib.import_module(f"landmarksystem_b200.models.{family}.{name}")
        trainer_cls = mod.NGPTrainer if family == "instant_ngp" else mod.NerfactoTrainer
        conf = os.path.join(ROOT, "landmarksystem_b200", "models", family, "confs", "synthetic_tiny.py")
        cfg = BaseConfig.from_file(conf, dict(over))
        if mode == "branch":
            cfg.branch_parallel, cfg.plane_division = True, [2, 1]
        else:
            cfg.DDP = True
        trainer = trainer_cls(cfg)
        trainer.train()
        first = next(iter(trainer.module.mlp_head.parameters())).detach().clone()
        queue.put((rank, None, (trainer.eval(), trainer.logfolder, first.numpy())))
    except Exception:
        queue.put((rank, traceback.format_exc(), None))


def _spawn_training(family, over, mode):
    ctx = mp.get_context("spawn")
    queue = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_train_worker, args=(r, 2, port, family, over, mode, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get() for _ in range(2)]
    for p in procs:
        p.join(timeout=180)
    for r in results:
        assert r[1] is None, r[1]
    return {r[0]: r[2] for r in results}


@pytest.mark.parametrize("family", ["instant_ngp", "nerfacto"])
def test_hash_models_train_in_parallel_on_cpu_ranks(family, tmp_path):
    """Spatial-block ("branch") parallel and data parallel training of the hash-grid models on two ranks (reference:
    instant_ngp_trainer.py:95-125, confs `*_BranchParallel.py` / `*_ddp*.py`).  Branch parallel: one table per rank, the
    merged checkpoint evaluates in ONE process to the PSNR the two ranks measured together.  Data parallel: the
    replicas hold identical weights after training."""
    import importlib

    import numpy as np

    from landmarksystem_b200.configs import BaseConfig

    over = {"basedir": str(tmp_path), "device": "cpu", "n_iters": "4", "datadir": "ring:4:12x12:14:3", "batch_size": "64",
            "progress_refresh_rate": "2", "N_vis": "-1"}
    if family == "instant_ngp":
        over["render_stratified_sampling"] = "False"
    else:
        over["use_proposal_weight_anneal"] = "False"      # the annealing exponent is trainer state, not checkpoint content
    out = _spawn_training(family, over, "branch")
    psnr, folder, _ = out[0]
    assert abs(out[1][0] - psnr) < 1e-6
    files = set(os.listdir(folder))
    assert {"state_dict-sub0.th", "state_dict-sub1.th", "state_dict-merged.th", "kwargs-merged.th"} <= files
    merged = torch.load(os.path.join(folder, "state_dict-merged.th"), weights_only=False)
    assert {"mlp_base_grid.tcnn_encoding.0.params", "mlp_base_grid.tcnn_encoding.1.params"} <= set(merged)

    name = "instant_ngp_evaluator" if family == "instant_ngp" else "nerfacto_evaluator"
    ev_mod = importlib.import_module(f"landmarksystem_b200.models.{family}.{name}")
    ev_cls = ev_mod.NGPEvaluator if family == "instant_ngp" else ev_mod.NerfactoEvaluator
    conf = os.path.join(ROOT, "landmarksystem_b200", "models", family, "confs", "synthetic_tiny.py")
    cfg = BaseConfig.from_file(conf, dict(over))
    cfg.update(is_train=False, plane_division=[2, 1], ckpt=os.path.join(folder, "state_dict-merged.th"),
               kwargs=os.path.join(folder, "kwargs-merged.th"), expname="merged_eval")
    alone = ev_cls(cfg).eval()
    assert abs(alone - psnr) < 1e-3, (alone, psnr)
    # ``ckpt="auto"`` finds the merged files of the run by its experiment name
    auto = BaseConfig.from_file(conf, dict(over))
    auto.update(is_train=False, plane_division=[2, 1], branch_parallel=True, ckpt="auto", ckpt_type="full")
    evaluator = ev_cls.__new__(ev_cls)
    evaluator.config, evaluator.logfolder = auto, folder
    evaluator.resolve_auto_ckpt()
    assert auto.ckpt == os.path.join(folder, "state_dict-merged.th") and auto.kwargs == os.path.join(folder, "kwargs-merged.th")

    out = _spawn_training(family, dict(over, expname="ddp_run"), "ddp")
    assert np.allclose(out[0][2], out[1][2], atol=1e-7) and abs(out[0][0] - out[1][0]) < 1e-6


def _grid_channel_worker(rank, world, port, over, queue):
    import traceback

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    try:
        from landmarksystem_b200.configs import BaseConfig
        from landmarksystem_b200.models.gridnerf.gridnerf_trainer import GridNeRFTrainer

        conf = os.path.join(ROOT, "landmarksystem_b200", "models", "gridnerf", "confs", "synthetic_tiny.py")
        cfg = BaseConfig.from_file(conf, dict(over))
        cfg.channel_parallel, cfg.channel_parallel_size = True, 2
        trainer = GridNeRFTrainer(cfg)
        trainer.train()
        queue.put((rank, None, (trainer.eval(), trainer.logfolder)))
    except Exception:
        queue.put((rank, traceback.format_exc(), None))


def test_channel_parallel_training_writes_a_merged_checkpoint(tmp_path):
    """Two ranks train GridNeRF with the feature channels split between them; rank 0 concatenates the slices into
    ``state_dict-merged.th`` / ``kwargs-merged.th`` (reference: gridnerf_trainer.py:488-504 - the shipped
    ``*_ChannelParallel_render.py`` configurations load exactly these files).  One process evaluating the merged files
    gets what one process gets from a run it trained alone with the same seed."""
    from landmarksystem_b200.configs import BaseConfig
    from landmarksystem_b200.models.gridnerf.gridnerf_evaluator import GridNeRFEvaluator
    from landmarksystem_b200.models.gridnerf.gridnerf_trainer import GridNeRFTrainer

    conf = os.path.join(ROOT, "landmarksystem_b200", "models", "gridnerf", "confs", "synthetic_tiny.py")
    over = {"basedir": str(tmp_path / "par"), "device": "cpu", "n_iters": "6", "datadir": "ring:4:12x12:14:3",
            "batch_size": "64", "progress_refresh_rate": "2", "N_vis": "-1", "nSamples": "24"}
    ctx = mp.get_context("spawn")
    queue = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_grid_channel_worker, args=(r, 2, port, over, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get() for _ in range(2)]
    for p in procs:
        p.join(timeout=180)
    for r in results:
        assert r[1] is None, r[1]
    parallel_psnr, folder = [r[2] for r in results if r[0] == 0][0]
    merged = torch.load(os.path.join(folder, "state_dict-merged.th"), weights_only=False)
    assert merged["density_encoding.plane_coef.0"].shape[1] == 16 and merged["rgb_encoding.line_coef.0"].shape[1] == 48
    part = torch.load(os.path.join(folder, "state_dict-sub1.th"), weights_only=False)
    assert part["density_encoding.plane_coef.0"].shape[1] == 8 and part["rgb_encoding.line_coef.0"].shape[1] == 24

    def evaluate(ckpt, kwargs, name):
        cfg = BaseConfig.from_file(conf, dict(over, basedir=str(tmp_path / name)))
        cfg.update(is_train=False, ckpt=ckpt, kwargs=kwargs, expname=name)
        return GridNeRFEvaluator(cfg).eval()

    from_merged = evaluate(os.path.join(folder, "state_dict-merged.th"), os.path.join(folder, "kwargs-merged.th"), "merged")
    alone = GridNeRFTrainer(BaseConfig.from_file(conf, dict(over, basedir=str(tmp_path / "alone"))))
    alone.train()
    assert abs(alone.eval() - parallel_psnr) < 1e-3                 # channel-parallel training follows the same trajectory
    from_alone = evaluate(os.path.join(alone.logfolder, "state_dict.th"), os.path.join(alone.logfolder, "kwargs.th"), "single")
    assert abs(from_merged - from_alone) < 1e-3, (from_merged, from_alone)

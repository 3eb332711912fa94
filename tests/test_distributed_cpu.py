"""Host-side distributed logic on CPU ranks (gloo, world size 2-4): group algebra, collective wrappers,
differentiable collectives, data-parallel and branch-parallel GridNeRF equivalence, failure detection."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from landmarksystem_b200.comm.group_initializer import (DPGroupInitializer, DynamicLoadGroupInitializer,
                                                        MessageTransferInitializer, TPGroupInitializer)
from landmarksystem_b200.comm.train_groups import group_layout


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(fn, world, *args):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get() for _ in range(world)]      # drain before joining: a full pipe blocks the writer
    for p in procs:
        p.join(timeout=120)
    for r in results:
        assert r[1] is None, r[1]
    return {r[0]: r[2] for r in results}


def _to_plain(obj):
    """Tensors leave the worker as numpy arrays (tensor pickling hands out shared-memory handles that die
    with the worker)."""
    if torch.is_tensor(obj):
        return obj.detach().cpu().numpy()
    if isinstance(obj, (tuple, list)):
        return type(obj)(_to_plain(o) for o in obj)
    return obj


def _entry(fn, rank, world, port, q, args):
    import traceback

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, None, _to_plain(out)))
    except Exception:
        q.put((rank, traceback.format_exc(), None))


# -- pure rank algebra -------------------------------------------------------------------------------
def test_render_group_layouts():
    assert DPGroupInitializer(0, 8, 4).layout() == [[0, 2, 4, 6]]
    assert TPGroupInitializer(0, 8, 2).layout() == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert MessageTransferInitializer(0, 4).layout() == [[0, 1, 2, 3]]
    # two nodes of 4 GPUs, tp=2: per node, ranks with the same tp offset
    assert DynamicLoadGroupInitializer(0, 8, 2, 4).layout() == [[0, 2], [4, 6], [1, 3], [5, 7]]


def test_train_group_layout():
    mp_groups, dp_groups = group_layout(8, 4)
    assert mp_groups == [[0, 1, 2, 3], [4, 5, 6, 7]] and dp_groups == [[0, 4], [1, 5], [2, 6], [3, 7]]


# -- collectives -----------------------------------------------------------------------------------------
def _collectives(rank, world):
    from landmarksystem_b200.comm import (CommContext, ParallelMode, all_gather, all_reduce, broadcast,
                                          broadcast_object_list, gather, scatter)
    from landmarksystem_b200.comm.autograd import AllGather, AllReduce
    from landmarksystem_b200.comm.varlen import all_gather_varlen
    from landmarksystem_b200.utils import Config

    ctx = CommContext()
    ctx.init_distributed_env(world_size=world, rank=rank, backend="gloo")
    ctx.init_groups(Config(tp_size=2))
    assert ctx.get_world_size(ParallelMode.TENSOR_PARALLEL) == 2
    x = torch.arange(5.0) + rank
    out = torch.empty(5 * world)
    all_gather(out, x)
    assert torch.equal(out, torch.cat([torch.arange(5.0) + r for r in range(world)]))
    y = x.clone()
    all_reduce(y)
    assert torch.equal(y, sum(torch.arange(5.0) + r for r in range(world)))
    b = x.clone()
    broadcast(b, src=1)
    assert torch.equal(b, torch.arange(5.0) + 1)
    box = [{"pose": [1, 2, 3]} if rank == 0 else None]
    broadcast_object_list(box, src=0)
    assert box[0] == {"pose": [1, 2, 3]}
    recv = torch.empty(5)
    scatter(recv, [torch.full((5,), float(r)) for r in range(world)] if rank == 0 else None, src=0)
    assert torch.equal(recv, torch.full((5,), float(rank)))
    lst = [torch.empty(5) for _ in range(world)] if rank == 0 else None
    gather(x, lst, dst=0)
    if rank == 0:
        assert torch.equal(lst[world - 1], torch.arange(5.0) + world - 1)
    # tensor-parallel group collectives touch only the pair
    t = torch.tensor([float(rank)])
    all_reduce(t, comm_mode=ParallelMode.TENSOR_PARALLEL)
    pair = (rank // 2) * 2
    assert float(t) == pair + pair + 1
    # differentiable collectives
    z = (torch.ones(3) * (rank + 1)).requires_grad_()
    g = AllGather.apply(z)
    (g * torch.arange(1.0, 3 * world + 1)).sum().backward()
    assert torch.equal(z.grad, torch.arange(1.0, 3 * world + 1)[rank * 3:(rank + 1) * 3])
    w = torch.ones(2, requires_grad=True)
    AllReduce.apply(w * (rank + 1)).sum().backward()
    assert torch.equal(w.grad, torch.full((2,), float(world * (rank + 1))))
    parts = all_gather_varlen(torch.full((rank + 1, 2), float(rank)))
    assert [p.shape[0] for p in parts] == list(range(1, world + 1)) and float(parts[-1][0, 0]) == world - 1
    ctx.destroy()
    return True


def test_collective_wrappers_gloo():
    _run(_collectives, 4)


# -- model-level equivalences ----------------------------------------------------------------------------------
def _make_model(division, branch, rank_cfg=None):
    from landmarksystem_b200.comm.train_groups import init_train_groups
    from landmarksystem_b200.components.scene import SceneManager
    from landmarksystem_b200.convertor import ComponentConvertorFactory
    from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF, GridNeRFConfig
    from landmarksystem_b200.utils import Config

    mc = GridNeRFConfig(resMode=[1], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0)
    cfg = Config(dict(mc))
    cfg.update(is_train=True, device="cpu", lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=division,
               branch_parallel=branch, channel_parallel=False, model_parallel_and_DDP=False, DDP=False)
    if branch:
        init_train_groups(cfg)
    sm = SceneManager(cfg)
    torch.manual_seed(0)
    model = GridNeRF(sm.aabb, [16 * division[0], 16 * division[1], 8], "cpu", near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    if branch:
        model = ComponentConvertorFactory.get_convertor("parallelize").convert(model, cfg)
    return model.eval(), cfg


def _rays(n=256):
    g = torch.Generator().manual_seed(5)
    o = torch.cat((torch.rand(n, 2, generator=g) * 3.6 - 1.8, torch.full((n, 1), 3.0)), -1)
    d = torch.nn.functional.normalize(torch.cat((torch.randn(n, 2, generator=g) * 0.3, -torch.ones(n, 1)), -1), dim=-1)
    return torch.cat((o, d, torch.zeros(n, 1)), -1)


def _branch_worker(rank, world, full_state):
    model, cfg = _make_model([2, 1], True)
    # give every rank its block of the single-process model, and the same heads
    for name in ("density_encoding", "rgb_encoding"):
        enc = getattr(model, name)
        enc.load_full_state({k[len(name) + 1:]: v for k, v in full_state.items() if k.startswith(name + ".")})
    heads = {k: v for k, v in full_state.items() if "encoding" not in k}
    model.load_state_dict(heads, strict=False)
    torch.manual_seed(11)
    out = model(_rays(), N_samples=32)["rgb_map"]
    out.sum().backward()
    g = model.density_encoding.plane_coef[0].grad
    return out.detach(), g.clone()


def test_branch_parallel_matches_single_process():
    single, _ = _make_model([2, 1], False)
    for p in single.density_encoding.parameters():
        p.data.abs_().mul_(2.0)
    state = {k: v.clone() for k, v in single.state_dict().items()}
    torch.manual_seed(11)
    ref = single(_rays(), N_samples=32)["rgb_map"]
    ref.sum().backward()
    res = _run(_branch_worker, 2, state)
    for r in (0, 1):
        assert torch.allclose(torch.from_numpy(res[r][0]), ref.detach(), atol=1e-5)
        assert torch.allclose(torch.from_numpy(res[r][1])[0], single.density_encoding.plane_coef[0].grad[r], atol=1e-5)


def _ddp_worker(rank, world, tmp):
    from landmarksystem_b200.configs import BaseConfig
    from landmarksystem_b200.models.gridnerf.gridnerf_trainer import GridNeRFTrainer

    conf = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "landmarksystem_b200", "models", "gridnerf",
                        "confs", "synthetic_tiny.py")
    cfg = BaseConfig.from_file(conf, {"basedir": tmp, "device": "cpu", "n_iters": "6", "batch_size": "256", "DDP": "true",
                                      "datadir": "ring:3:16x16:20:3", "nSamples": "24", "progress_refresh_rate": "100"})
    tr = GridNeRFTrainer(cfg)
    tr.model.train()
    for it in range(6):
        tr.train_step(*tr.data_mgr.get_rays(it))
    flat = torch.cat([p.detach().reshape(-1) for p in tr.module.parameters()])
    return flat


def test_data_parallel_replicas_stay_identical(tmp_path):
    res = _run(_ddp_worker, 2, str(tmp_path))
    assert torch.allclose(torch.from_numpy(res[0]), torch.from_numpy(res[1]), atol=1e-6)


def _channel_model(parallel: bool):
    from landmarksystem_b200.comm.train_groups import init_train_groups
    from landmarksystem_b200.components.scene import SceneManager
    from landmarksystem_b200.convertor import ComponentConvertorFactory
    from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF, GridNeRFConfig
    from landmarksystem_b200.utils import Config

    mc = GridNeRFConfig(resMode=[1, 2], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0)
    cfg = Config(dict(mc))
    cfg.update(is_train=True, device="cpu", lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=[1, 1],
               branch_parallel=False, channel_parallel=parallel, channel_parallel_size=2 if parallel else 1,
               model_parallel_and_DDP=False, DDP=False)
    if parallel:
        init_train_groups(cfg)
    sm = SceneManager(cfg)
    torch.manual_seed(0)
    model = GridNeRF(sm.aabb, [16, 16, 8], "cpu", near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    if parallel:
        model = ComponentConvertorFactory.get_convertor("parallelize").convert(model, cfg)
    return model.train(), cfg


def _train_three_steps(model):
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    target = torch.rand(256, 3, generator=torch.Generator().manual_seed(9))
    for k in range(3):
        torch.manual_seed(100 + k)                      # same sample jitter / background draw everywhere
        out = model(_rays(), N_samples=24)["rgb_map"]
        loss = ((out - target) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
    return float(loss)


def _channel_worker(rank, world, full_state):
    model, cfg = _channel_model(True)
    for name in ("density_encoding", "rgb_encoding"):
        getattr(model, name).load_full_state({k[len(name) + 1:]: v for k, v in full_state.items() if k.startswith(name + ".")})
    model.load_state_dict({k: v for k, v in full_state.items() if "encoding" not in k}, strict=False)
    loss = _train_three_steps(model)
    planes = [p.detach().clone() for p in model.rgb_encoding.plane_coef] + [p.detach().clone() for p in model.density_encoding.plane_coef]
    head = model.rgb_decoder.decoder.linears()[0].weight.detach().clone()
    return loss, planes, head


def test_channel_parallel_training_matches_single_process():
    """Three Adam steps with the feature channels split over two ranks (each rank trains its channel slice of every
    plane and line, the replicated heads see the gathered features) against the same three steps in one process."""
    single, _ = _channel_model(False)
    state = {k: v.clone() for k, v in single.state_dict().items()}
    want_loss = _train_three_steps(single)
    res = _run(_channel_worker, 2, state)
    want_planes = [p.detach() for p in single.rgb_encoding.plane_coef] + [p.detach() for p in single.density_encoding.plane_coef]
    for k, want in enumerate(want_planes):
        got = torch.cat([torch.from_numpy(res[r][1][k]) for r in range(2)], dim=-1)     # channel slices side by side
        assert got.shape == want.shape
        assert torch.allclose(got, want, atol=2e-5), (k, float((got - want).abs().max()))
    for r in range(2):
        assert abs(res[r][0] - want_loss) < 1e-5
        assert torch.allclose(torch.from_numpy(res[r][2]), single.rgb_decoder.decoder.linears()[0].weight.detach(), atol=2e-5)


def _hybrid_worker(rank, world, tmp):
    from landmarksystem_b200.configs import BaseConfig
    from landmarksystem_b200.models.gridnerf.gridnerf_trainer import GridNeRFTrainer

    conf = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "landmarksystem_b200", "models", "gridnerf",
                        "confs", "synthetic_tiny.py")
    cfg = BaseConfig.from_file(conf, {"basedir": tmp, "device": "cpu", "n_iters": "4", "batch_size": "256", "DDP": "true",
                                      "branch_parallel": "true", "model_parallel_and_DDP": "true",
                                      "datadir": "ring:3:16x16:20:3", "nSamples": "24", "progress_refresh_rate": "100"})
    cfg.plane_division = [2, 1]
    tr = GridNeRFTrainer(cfg)
    tr.model.train()
    for it in range(4):
        tr.train_step(*tr.data_mgr.get_rays(it))
    grids = torch.cat([p.detach().reshape(-1) for n, p in tr.module.named_parameters() if "encoding" in n])
    heads = torch.cat([p.detach().reshape(-1) for n, p in tr.module.named_parameters() if "encoding" not in n])
    return int(cfg.mp_rank), int(cfg.dp_rank), grids, heads


def test_hybrid_model_and_data_parallel_groups_train_consistently(tmp_path):
    """Four ranks = 2 spatial blocks x 2 data-parallel replicas (contiguous model-parallel groups, strided data-parallel
    groups; reference layout: landmark/nerf_components/components_convertor/comm_groups.py:51-75).  After four steps the
    two replicas of each block hold identical grids, every rank holds identical heads, and the two blocks differ."""
    res = _run(_hybrid_worker, 4, str(tmp_path))
    by = {(res[r][0], res[r][1]): (torch.from_numpy(res[r][2]), torch.from_numpy(res[r][3])) for r in range(4)}
    assert sorted(by) == [(0, 0), (0, 1), (1, 0), (1, 1)]
    for mp in (0, 1):
        assert torch.allclose(by[(mp, 0)][0], by[(mp, 1)][0], atol=1e-6)
    assert not torch.allclose(by[(0, 0)][0], by[(1, 0)][0], atol=1e-3)
    for key in by:
        assert torch.allclose(by[key][1], by[(0, 0)][1], atol=1e-6)


# -- data-parallel render: rows dealt round-robin (or in bands), results back in the original order --------------------
def _dp_scatter_gather(rank, world):
    from landmarksystem_b200.comm import CommContext
    from landmarksystem_b200.render.parallel_module import ParallelModule, StageArgs
    from landmarksystem_b200.utils import Config

    ctx = CommContext()
    ctx.init_distributed_env(world_size=world, rank=rank, backend="gloo")
    ctx.init_groups(Config(tp_size=1))

    class Plain(ParallelModule):
        def _parallize(self, model):
            return model

    rows = torch.arange(11.0)[:, None].repeat(1, 2)                 # 11 rows: padded to 12 for 2 and for 4 ranks
    parts = {}
    for interleave in (True, False):
        pm = Plain(torch.nn.Identity(), Config(parallel_config=Config(tp_size=1, dp_interleave=interleave)))
        args, _ = pm.dp_scatter(StageArgs((rows,), {}))
        assert args[0].shape[0] == 12 // world
        res, _ = pm.dp_gather(StageArgs((args[0] * 2.0, "kept"), {}))
        assert torch.equal(res[0], rows * 2.0) and res[1] == "kept"
        parts[interleave] = args[0][:, 0].tolist()
    ctx.destroy()
    return parts


@pytest.mark.parametrize("world", [2, 4])
def test_data_parallel_render_scatter_gather(world):
    out = _run(_dp_scatter_gather, world)
    size = 12 // world
    for rank in range(world):
        padded = list(range(11)) + [0]
        assert [int(v) for v in out[rank][True]] == padded[rank::world]
        assert [int(v) for v in out[rank][False]] == padded[rank * size:(rank + 1) * size]


# -- the engine's user-input message: one fixed-size broadcast, object broadcast for what does not fit ------------------
def _user_inputs(rank, world):
    from landmarksystem_b200.comm import CommContext
    from landmarksystem_b200.comm.collective import _broadcast_user_inputs_message
    from landmarksystem_b200.utils import Config

    ctx = CommContext()
    ctx.init_distributed_env(world_size=world, rank=rank, backend="gloo")
    ctx.init_groups(Config(tp_size=1))
    small = [(torch.arange(16.0).reshape(4, 4), 262144, 1080, 1920, 2317.6), {"app_code": 3}]
    got = _broadcast_user_inputs_message(small if rank == 0 else None)
    assert torch.equal(got[0][0], small[0][0]) and got[0][1:] == small[0][1:] and got[1] == small[1]
    big = [(torch.arange(50000.0),), {}]                     # 200 KB: does not fit the fixed buffer
    got_big = _broadcast_user_inputs_message(big if rank == 0 else None)
    assert torch.equal(got_big[0][0], big[0][0])
    got = _broadcast_user_inputs_message(small if rank == 0 else None)       # and the fast path again afterwards
    assert got[0][2] == 1080
    ctx.destroy()
    return True


def test_engine_user_inputs_broadcast():
    _run(_user_inputs, 2)


def _module_level_groups(rank, world):
    from landmarksystem_b200.train import utils as tu

    assert tu.is_dist_avail_and_initialized() and tu.is_main_process() == (rank == 0)
    tu.init_comm_groups(model_parallel_degree=2)
    mp = torch.tensor([float(rank)])
    dist.all_reduce(mp, group=tu.get_mp_group())            # ranks {0,1} and {2,3}
    dp = torch.tensor([float(rank)])
    dist.all_reduce(dp, group=tu.get_dp_group())            # ranks {0,2} and {1,3}
    return float(mp), float(dp), tu.get_mp_rank0(), tu.get_mp_part()


def test_module_level_group_helpers():
    """``init_comm_groups / get_dp_group / get_mp_group / get_mp_rank0 / get_mp_part`` of the reference's
    ``distributed_utils`` (world 4, model-parallel degree 2)."""
    out = _run(_module_level_groups, 4)
    assert out[0] == (1.0, 2.0, 0, 0) and out[1] == (1.0, 4.0, 0, 1)
    assert out[2] == (5.0, 2.0, 2, 0) and out[3] == (5.0, 4.0, 2, 1)


def test_print_silencer_and_save_on_master(tmp_path, capsys):
    import builtins

    from landmarksystem_b200.train import utils as tu

    original = tu.setup_for_distributed(False)
    try:
        print("hidden")
        print("shown", force=True)
    finally:
        builtins.print = original
    assert capsys.readouterr().out == "shown\n"
    tu.save_on_master({"a": 1}, str(tmp_path / "x.th"))     # single process: rank 0
    assert torch.load(str(tmp_path / "x.th"), weights_only=False) == {"a": 1} and tu.get_local_size() == 1

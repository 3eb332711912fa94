"""Rendering engine: schedules, init_inference round trip, dynamic loading and the stage pipeline."""
import os

import numpy as np
import pytest
import torch

import landmarksystem_b200 as lm
from landmarksystem_b200.components.scene import SceneManager
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF, GridNeRFConfig
from landmarksystem_b200.render.adapters import make_adapter
from landmarksystem_b200.render.easy_pipeline import EasyPipeRunner, PipelineItem
from landmarksystem_b200.render.offload.utils import calculate_block_neighbours
from landmarksystem_b200.render.sches import DDPSche, InferenceSche, MultiDeviceSche, gen_scheduler
from landmarksystem_b200.synthetic import look_at
from landmarksystem_b200.utils import Config


def _model_config(tmp_path, division, device="cpu", **extra):
    mc = GridNeRFConfig(resMode=[1, 2], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0, n_importance=48, sampling_opt=True)
    cfg = Config(dict(mc))
    cfg.update(is_train=False, device=device, lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=division,
               branch_parallel=False, ckpt=str(tmp_path / "state_dict.th"), kwargs=str(tmp_path / "kwargs.th"), **extra)
    return cfg


def _save_random_model(tmp_path, division):
    torch.manual_seed(0)
    cfg = _model_config(tmp_path, division)
    sm = SceneManager(cfg)
    model = GridNeRF(sm.aabb, [32 * division[0], 32 * division[1], 16], "cpu", near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    for p in model.density_encoding.parameters():
        p.data.abs_().mul_(3.0)       # make the random field visibly dense
    model.save_model(str(tmp_path))
    return model


def _pose(x, y):
    return look_at(torch.tensor([x, y, 3.0]), torch.tensor([x + 0.05, y, 0.0]), up=(0.0, 1.0, 0.0))


def test_schedules():
    assert InferenceSche().steps()[1].__name__ == "PreprocessInstruction"
    assert "BroadcastInputsInstruction" in [s.__name__ for s in MultiDeviceSche().steps()]
    names = [s.__name__ for s in DDPSche().steps()]
    assert names.index("DPScatterInstruction") < names.index("CallInstruction") < names.index("DPGatherInstruction")
    assert isinstance(gen_scheduler(Config(runtime="Torch")), InferenceSche)


def test_block_neighbours():
    assert calculate_block_neighbours(0, [4, 4], [3, 3]) == [0, 1, 2, 4, 5, 6, 8, 9, 10]
    assert calculate_block_neighbours(15, [4, 4], [2, 2]) == [10, 11, 14, 15]
    assert calculate_block_neighbours(5, [4, 4], [1, 1]) == [5]
    assert calculate_block_neighbours(3, [2, 2], [3, 3]) == [0, 1, 2, 3]


def test_sanity_checks():
    with pytest.raises(AssertionError):
        lm._infer_config_sanity_check(Config(act_cache=True), Config(offload_config={"local_plane_split": [1, 1]}))
    with pytest.raises(AssertionError):
        lm._infer_config_sanity_check(Config(), Config(offload_config={}, parallel_config={"tp_size": 2}))
    with pytest.raises(AssertionError):
        lm._infer_config_sanity_check(Config(), Config(half_precision=True))


def _engine(tmp_path, division, device, **inference):
    cfg = _model_config(tmp_path, division, device)
    inf = Config(runtime="Torch", kernel_fusion=False, **inference)
    return lm.init_inference(GridNeRF, make_adapter(GridNeRF), cfg, inf)


def _render_pair(tmp_path, device):
    direct = _save_random_model(tmp_path, [2, 2])
    engine = _engine(tmp_path, [2, 2], device)
    img, depth = engine(_pose(-0.9, 0.8), 4096, 24, 32, 30.0)
    assert img.shape == (24, 32, 4) and img.dtype == torch.uint8 and depth.shape == (24, 32)
    # same pixels as calling the model directly
    mod = make_adapter(GridNeRF)
    adapter = object.__new__(mod)
    torch.nn.Module.__init__(adapter)
    adapter.model, adapter.scene_mgr = direct, None
    (rays,), _ = adapter.preprocess(_pose(-0.9, 0.8), 4096, 24, 32, 30.0)
    direct.eval()
    ref = direct.render_all_rays(rays, chunk_size=4096)["rgb_map"].clamp(0, 1).reshape(24, 32, 3)
    assert (img[..., :3].float().cpu() - ref * 255).abs().max() <= 2.0
    return img


def test_init_inference_matches_direct_render_cpu(tmp_path):
    img = _render_pair(tmp_path, "cpu")
    assert img[..., :3].float().std() > 1.0          # not a constant image


def test_dynamic_loading_matches_full_model_cpu(tmp_path):
    _save_random_model(tmp_path, [2, 2])
    full = _engine(tmp_path, [2, 2], "cpu")
    off = _engine(tmp_path, [2, 2], "cpu", offload_config={"local_plane_split": [1, 1], "plane_split": [2, 2]})
    # the camera visits every block; a 1x1 window only shows the block under the camera, so compare
    # on rays that stay inside that block (narrow field of view, looking straight down)
    for x, y in ((-1.0, -1.0), (-1.0, 1.0), (1.0, 1.0), (1.0, -1.0), (-1.0, -1.0)):
        a, _ = full(_pose(x, y), 4096, 16, 16, 120.0)
        b, _ = off(_pose(x, y), 4096, 16, 16, 120.0)
        assert (a.float() - b.float()).abs().max() <= 2.0
    mgr = off.model.model.buffer_manager
    assert mgr.bytes_h2d > 0 and len(mgr.get_buffer().local_block_idxes) == 1


def test_channel_last_checkpoint_renders_like_the_original(tmp_path):
    """``transform_gridnerf_model_to_channel_last`` writes ``*_channel_last.th`` with planes stored ``[1, B, H, W, C]``
    (reference: landmark/render/util/utils.py:6-19, tests/test_module/test_util/test_channel_last_transform.py); the
    engine renders the same image from either file, resident or under dynamic loading with ``channel_last=True``."""
    from landmarksystem_b200.render.utils import transform_gridnerf_model_to_channel_last

    _save_random_model(tmp_path, [2, 2])
    original = torch.load(str(tmp_path / "state_dict.th"), weights_only=False)
    out = transform_gridnerf_model_to_channel_last(str(tmp_path / "state_dict.th"))
    assert out.endswith("state_dict_channel_last.th")
    moved = torch.load(out, weights_only=False)
    key = "density_encoding.plane_coef.0"
    assert moved[key].shape == tuple(original[key].shape[i] for i in (0, 2, 3, 4, 1))
    assert torch.equal(moved[key].permute(0, 4, 1, 2, 3), original[key])
    assert torch.equal(moved["density_encoding.line_coef.0"], original["density_encoding.line_coef.0"])

    def engine(ckpt, **inference):
        cfg = _model_config(tmp_path, [2, 2], "cpu")
        cfg.ckpt = ckpt
        return lm.init_inference(GridNeRF, make_adapter(GridNeRF), cfg, Config(runtime="Torch", kernel_fusion=False, **inference))

    want, _ = engine(str(tmp_path / "state_dict.th"))(_pose(-0.9, 0.8), 4096, 16, 16, 60.0)
    got, _ = engine(out)(_pose(-0.9, 0.8), 4096, 16, 16, 60.0)
    assert torch.equal(got, want) and want[..., :3].float().std() > 1.0
    window = {"local_plane_split": [2, 2], "plane_split": [2, 2], "channel_last": True}
    streamed, _ = engine(out, offload_config=window)(_pose(-0.9, 0.8), 4096, 16, 16, 60.0)
    assert (streamed.float() - want.float()).abs().max() <= 1.0


def test_dynamic_loading_window_reuses_resident_blocks(tmp_path):
    _save_random_model(tmp_path, [2, 2])
    off = _engine(tmp_path, [2, 2], "cpu", offload_config={"local_plane_split": [2, 1], "plane_split": [2, 2]})
    off(_pose(-1.0, -1.0), 4096, 8, 8, 60.0)
    mgr = off.model.model.buffer_manager
    first = mgr.bytes_h2d
    off(_pose(-1.0, 1.0), 4096, 8, 8, 60.0)       # window [1, 3]: nothing shared with [0, 2]
    off(_pose(-1.0, 1.0), 4096, 8, 8, 60.0)
    assert mgr.get_buffer().local_block_idxes == [1, 3] and mgr.bytes_h2d == 2 * first


def _ngp_config(tmp_path, division, **extra):
    from landmarksystem_b200.models.instant_ngp.instant_ngp import InstantNGPConfig

    mc = InstantNGPConfig(num_levels=4, base_res=8, max_res=64, log2_hashmap_size=12, grid_resolution=16, grid_levels=1,
                          train_near_far=[0.5, 6.0], appearance_embedding_size=4, render_step_size=0.05, cone_angle=0.0,
                          max_samples_per_ray=96, background_color="black", runtime="Torch",
                          render_stratified_sampling=False)
    cfg = Config(dict(mc))
    cfg.update(is_train=False, device="cpu", lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=division,
               branch_parallel=False, ckpt=str(tmp_path / "state_dict.th"), kwargs=str(tmp_path / "kwargs.th"),
               aabb_norm_range=[0, 1], **extra)
    return cfg


def test_dynamic_loading_of_a_hash_table_model_matches_the_full_model(tmp_path):
    """InstantNGP with one hash table per block (the reference tests this combination with a [1, 2] window,
    tests/test_inference_framework/test_single_device/test_torch_inference.py:210-319): a 1x1 window follows the camera
    over all four blocks; the tables of the window sit in window order, so samples are routed by window-relative ids."""
    from landmarksystem_b200.models.instant_ngp.instant_ngp import InstantNGP, window_remap
    from landmarksystem_b200.ops.ngp_field import sample_positions

    torch.manual_seed(0)
    cfg = _ngp_config(tmp_path, [2, 2])
    sm = SceneManager(cfg)
    model = InstantNGP(sm.aabb, "cpu", [0.5, 6.0], scene_manager=sm, config=cfg)
    for p in model.mlp_base_grid.parameters():
        p.data.normal_(0, 1.0)                      # a visibly structured random field, different in every block
    for head in (model.mlp_base_mlp, model.mlp_head):
        for p in head.parameters():
            p.data.mul_(4.0)
    model.save_model(str(tmp_path))
    full = lm.init_inference(InstantNGP, make_adapter(InstantNGP), _ngp_config(tmp_path, [2, 2]), Config(runtime="Torch"))
    off = lm.init_inference(InstantNGP, make_adapter(InstantNGP), _ngp_config(tmp_path, [2, 2]),
                            Config(runtime="Torch", offload_config={"local_plane_split": [1, 1], "plane_split": [2, 2]}))
    images = []
    for x, y in ((-1.0, -1.0), (-1.0, 1.0), (1.0, 1.0), (1.0, -1.0)):
        a, _ = full(_pose(x, y), 4096, 16, 16, 120.0)
        b, _ = off(_pose(x, y), 4096, 16, 16, 120.0)
        assert torch.equal(a, b) and a[..., :3].float().std() > 1.0
        images.append(a)
    assert not torch.equal(images[0], images[2])    # the blocks really hold different content
    stats = off.model.model.stats()
    assert stats["frames"] == 4 and stats["bytes_h2d"] > 0

    # rows of the position kernel's layout (row-major block id in the last column) remapped to the window
    inner = off.model.model.inner
    o = torch.tensor([[1.0, -1.0, 3.0]]).repeat(8, 1)
    d = torch.nn.functional.normalize(torch.tensor([[0.02 * k - 0.07, 0.3 * (k % 3) - 0.3, -1.0] for k in range(8)]), dim=-1)
    z = torch.linspace(2.6, 3.4, 8 * 4)
    xyzb, inside = sample_positions(None, 4, o, d, z, inner.aabb, None, 2, 2)
    got, keep = window_remap(inner.scene_manager, xyzb, inside, 2, 2)
    pos = (o[:, None] + d[:, None] * z.view(8, 4)[..., None]).reshape(-1, 3)
    want, want_keep = inner._positions(pos)
    assert torch.equal(keep, want_keep) and torch.allclose(got, want, atol=1e-6) and keep.any() and not keep.all()


def test_dynamic_loading_of_nerfacto_matches_the_full_model(tmp_path):
    """Nerfacto (contracted scene, proposal networks that stay resident, one field table per block) under a 1x1 window."""
    from landmarksystem_b200.models.nerfacto.nerfacto import Nerfacto, NerfactoConfig

    def config(**extra):
        mc = NerfactoConfig(num_levels=4, base_res=8, max_res=64, log2_hashmap_size=12, hidden_dim=32, hidden_dim_color=32,
                            appearance_embedding_size=4, num_proposal_samples_per_ray=(32, 16), num_nerf_samples_per_ray=12,
                            proposal_net_args_list=[{"hidden_dim": 16, "log2_hashmap_size": 10, "num_levels": 3, "max_res": 32},
                                                    {"hidden_dim": 16, "log2_hashmap_size": 10, "num_levels": 3, "max_res": 64}],
                            train_near_far=[0.5, 6.0], background_color="black", runtime="Torch")
        cfg = Config(dict(mc))
        cfg.update(is_train=False, device="cpu", lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=[2, 2],
                   branch_parallel=False, ckpt=str(tmp_path / "state_dict.th"), kwargs=str(tmp_path / "kwargs.th"),
                   aabb_norm_range=[0, 1], **extra)
        return cfg

    torch.manual_seed(0)
    cfg = config()
    sm = SceneManager(cfg)
    model = Nerfacto(sm.aabb, "cpu", [0.5, 6.0], scene_manager=sm, config=cfg)
    for p in model.mlp_base_grid.parameters():
        p.data.normal_(0, 1.0)
    model.save_model(str(tmp_path))
    full = lm.init_inference(Nerfacto, make_adapter(Nerfacto), config(), Config(runtime="Torch"))
    off = lm.init_inference(Nerfacto, make_adapter(Nerfacto), config(),
                            Config(runtime="Torch", offload_config={"local_plane_split": [1, 1], "plane_split": [2, 2]}))
    for x, y in ((-1.0, -1.0), (1.0, 1.0), (-1.0, 1.0)):
        a, _ = full(_pose(x, y), 4096, 12, 12, 120.0)
        b, _ = off(_pose(x, y), 4096, 12, 12, 120.0)
        assert torch.equal(a, b)
    mgr = off.model.model.buffer_manager
    assert len(mgr.get_buffer().local_block_idxes) == 1 and off.model.model.stats()["bytes_h2d"] > 0


def test_user_defined_model_and_adapter_through_init_inference():
    """A model and an inference module written by a user of the framework: no configuration, no checkpoint - the
    reference's engine smoke test (tests/test_inference_framework/test_inference.py:389-393, tests/utils.py:15-31)."""
    from landmarksystem_b200 import InferenceEngine, InferenceModule
    from landmarksystem_b200.components.model.base_model import BaseNeRF

    class SimpleModel(BaseNeRF):
        def __init__(self, N=10):
            super().__init__()
            self.layer1 = torch.nn.Linear(N, N)
            self.layer2 = torch.nn.ReLU()

        @staticmethod
        def get_kwargs():
            return {"N": 10}

        def forward(self, x):
            return self.layer2(self.layer1(x))

    class Doubling(InferenceModule):
        def __init__(self, **kwargs):
            super().__init__(SimpleModel(**kwargs))

        def preprocess(self, x, scale=1.0):
            return (x * scale,), {}

        def forward(self, x):
            return self.model(x)

        def postprocess(self, y):
            return {"doubled": 2.0 * y}

    torch.manual_seed(0)
    cfg = dict(runtime="Torch", kernel_fusion=False, ckpt_path=None)
    bare = lm.init_inference(SimpleModel, None, None, dict(cfg))
    assert isinstance(bare, InferenceEngine)
    x = torch.ones(10, 10)
    assert bare(x).shape == (10, 10) and float(bare(x).min()) >= 0
    engine = lm.init_inference(SimpleModel, Doubling, None, dict(cfg))
    inner = [m for m in engine.modules() if isinstance(m, SimpleModel)][0]
    out = engine(x, scale=3.0)
    assert set(out) == {"doubled"} and torch.allclose(out["doubled"], 2.0 * inner(3.0 * x))


def test_easy_pipeline_orders_results_and_reports_errors():
    runner = EasyPipeRunner([PipelineItem(lambda x: x + 1), PipelineItem(lambda x: x * 2)])
    runner.run_batch([1, 2, 3])
    assert [runner.get_result() for _ in range(3)] == [4, 6, 8]
    runner.run_batch(["boom"])
    with pytest.raises(TypeError):
        runner.get_result()
    runner.stop()


def test_easy_pipeline_worker_resources_and_queue_access():
    """A stage with ``init_fn`` owns a resource built once per worker; the reference's queue-level calls
    (``get_result_task``, ``get_result_queue``, ``wait_stop``) work on the same runner."""
    from landmarksystem_b200.render.easy_pipeline import SimpleWorker, Worker

    built = []

    def make_resource():
        built.append(1)
        return {"offset": 100}

    assert issubclass(SimpleWorker, Worker)
    runner = EasyPipeRunner([PipelineItem(lambda res, x: x + res["offset"], init_fn=make_resource),
                             PipelineItem(lambda x: -x)])
    assert runner.get_result_task(block=False) is None
    runner.run_batch([1, 2])
    first = runner.get_result_task(block=True)
    assert first.payload == -101 and runner.get_result() == -102 and built == [1]
    assert runner.pipeline.get_result_queue() is runner.result_queue
    runner.stop()
    runner.wait_stop()
    assert not any(t.is_alive() for t in runner.pipeline.threads)


@pytest.mark.gpu
def test_init_inference_kernel_runtime_gpu(tmp_path):
    _save_random_model(tmp_path, [2, 2])
    torch_engine = _engine(tmp_path, [2, 2], "cuda")
    cfg = _model_config(tmp_path, [2, 2], "cuda")
    kernel_engine = lm.init_inference(GridNeRF, make_adapter(GridNeRF), cfg, Config(runtime="Kernel", kernel_fusion=True))
    a, _ = torch_engine(_pose(-0.9, 0.8), 4096, 48, 64, 60.0)
    b, _ = kernel_engine(_pose(-0.9, 0.8), 4096, 48, 64, 60.0)
    assert (a.float() - b.float()).abs().mean() < 3.0      # bf16 grids + bf16 tensor-core MLP vs fp32


@pytest.mark.gpu
def test_dynamic_loading_gpu_bf16_stream(tmp_path):
    _save_random_model(tmp_path, [2, 2])
    full = _engine(tmp_path, [2, 2], "cuda")
    off = _engine(tmp_path, [2, 2], "cuda", offload_config={"local_plane_split": [1, 1], "plane_split": [2, 2], "dtype": "bf16"})
    for x, y in ((-1.0, -1.0), (1.0, 1.0), (1.0, 1.0), (1.0, 1.0)):
        a, _ = full(_pose(x, y), 4096, 16, 16, 120.0)
        b, _ = off(_pose(x, y), 4096, 16, 16, 120.0)
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().mean() < 3.0


def test_dynamic_loading_prefetches_ahead_of_a_scripted_camera_track(tmp_path):
    """A camera flies along +x over a 6x6-block scene with a 3x3 window.  With ``prefetch_frames`` the window is
    re-centred on the block the camera is about to enter BEFORE it crosses the boundary; without it (the reference's
    policy) the window only follows after the crossing.  No frame stalls in either case at this speed."""
    _save_random_model(tmp_path, [6, 6])
    width = 4.0 / 6.0                                  # block width of the [-2, 2] scene

    def fly(prefetch):
        off = _engine(tmp_path, [6, 6], "cpu", offload_config={"local_plane_split": [3, 3], "plane_split": [6, 6],
                                                             "prefetch_frames": prefetch, "swap_delay": 0})
        module = off.model.model
        centre_ahead = 0
        for k in range(60):
            x = -2.0 + width * 1.5 + 0.04 * k          # starts in the middle of block column 1, 0.06 blocks per frame
            off(_pose(x, 0.1), 4096, 4, 4, 60.0)
            col_now = int((x + 2.0) // width)
            window = module.buffer_manager.get_buffer().local_block_idxes
            cols = sorted({b // 6 for b in window})
            assert col_now in cols
            if len(cols) == 3 and cols[1] == col_now + 1:
                centre_ahead += 1                      # window already centred on the next column
        return module.stats(), centre_ahead

    stats, ahead = fly(8)
    assert stats["stalled_frames"] == 0 and stats["late_swaps"] == 0 and stats["frames"] == 60
    assert ahead > 0
    stats0, ahead0 = fly(0)
    assert stats0["stalled_frames"] == 0 and ahead0 == 0


def test_runtime_convertor_takes_a_state_dict_and_reports_swaps(tmp_path, capsys):
    """``convert(model, config, state_dict, verbose)`` as the reference calls it (convertor_factory.py:77-127)."""
    from landmarksystem_b200.components.fields.fused_mlp_decoder import FusedMLPDecoder
    from landmarksystem_b200.convertor import ComponentConvertorFactory

    source = _save_random_model(tmp_path, [1, 1])
    cfg = _model_config(tmp_path, [1, 1])
    sm = SceneManager(cfg)
    torch.manual_seed(5)
    fresh = GridNeRF(sm.aabb, [32, 32, 16], "cpu", near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
    state = torch.load(str(tmp_path / "state_dict.th"), weights_only=False)
    converted = ComponentConvertorFactory.get_convertor(convert_type="runtime").convert(fresh, cfg, state, True)
    printed = capsys.readouterr().out
    assert "->" in printed and any(isinstance(m, FusedMLPDecoder) for m in converted.modules())
    for (name, a), (_, b) in zip(source.state_dict().items(), converted.state_dict().items()):
        assert torch.allclose(a, b), name

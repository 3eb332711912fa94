"""Worker (2, 4 or 8 GPUs): ``init_inference`` with ``parallel_config = {"tp_size": world, "mode": "block"}``.  Each rank keeps one
rectangle of the scene's blocks; the engine broadcasts the pose, both ranks render their ray segments and the cross-GPU
composite merges them.  The image is compared with a single-process render of the same checkpoint."""
import json
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import landmarksystem_b200 as lm  # noqa: E402
from landmarksystem_b200.components.scene import SceneManager  # noqa: E402
from landmarksystem_b200.models.gridnerf.gridnerf import GridNeRF, GridNeRFConfig  # noqa: E402
from landmarksystem_b200.render.adapters import make_adapter  # noqa: E402
from landmarksystem_b200.synthetic import look_at  # noqa: E402
from landmarksystem_b200.utils import Config  # noqa: E402


def model_config(root, division, device):
    mc = GridNeRFConfig(resMode=[1], n_lamb_sigma=[16], n_lamb_sh=[48], nonlinear_density=True, view_pe=2, fea_pe=2,
                        train_near_far=[0.5, 6.0], step_ratio=2.0, sampling_opt=False, fea2denseAct="relu")
    cfg = Config(dict(mc))
    cfg.update(is_train=False, device=device, lb=[-2.0, -2.0, -0.5], ub=[2.0, 2.0, 0.5], plane_division=division,
               branch_parallel=False, ckpt=os.path.join(root, "state_dict.th"), kwargs=os.path.join(root, "kwargs.th"))
    return cfg


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    world = int(os.environ["WORLD_SIZE"])
    root = os.path.join(tempfile.gettempdir(), f"lmb_engine_block_mp_{world}")
    division = {2: [2, 2], 4: [2, 2], 8: [2, 4]}[world]      # 2 ranks: a band of two blocks each; 4 and 8: one block each
    if rank == 0:
        os.makedirs(root, exist_ok=True)
        torch.manual_seed(0)
        cfg = model_config(root, division, "cpu")
        sm = SceneManager(cfg)
        model = GridNeRF(sm.aabb, [32 * division[0], 32 * division[1], 16], "cpu", near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
        for p in model.density_encoding.parameters():
            p.data.abs_().mul_(3.0)
        model.save_model(root)
    # the engine initialises the process group itself (env:// rendezvous); wait for the checkpoint through the file system
    import time
    for _ in range(600):
        if os.path.exists(os.path.join(root, "kwargs.th")) and os.path.exists(os.path.join(root, "state_dict.th")):
            break
        time.sleep(0.1)
    time.sleep(0.5)
    dev = f"cuda:{int(os.environ['LOCAL_RANK'])}"
    engine = lm.init_inference(GridNeRF, make_adapter(GridNeRF), model_config(root, division, dev),
                               Config(runtime="Torch", kernel_fusion=False, parallel_config={"tp_size": world, "mode": "block"}))
    pose = look_at(torch.tensor([0.2, -0.1, 3.0]), torch.tensor([0.25, -0.1, 0.0]), up=(0.0, 1.0, 0.0))
    H, W = 48, 64
    out = engine(pose, 2048, H, W, 60.0) if rank == 0 else engine()
    if rank == 0:
        image = out[0] if isinstance(out, tuple) else out
        cfg = model_config(root, division, dev)
        ref_engine_cfg = Config(runtime="Torch", kernel_fusion=False)
        # single-process reference on this GPU: load the same checkpoint directly
        from landmarksystem_b200.render.initializer import InferenceModuleInitializer  # noqa: F401
        sm = SceneManager(cfg)
        kwargs = torch.load(cfg.kwargs, weights_only=False)
        ref = GridNeRF(sm.aabb, kwargs["gridSize"], dev, near_far=[0.5, 6.0], scene_manager=sm, config=cfg)
        ref.load_state_dict(torch.load(cfg.ckpt, weights_only=False))
        ref = ref.to(dev).eval()
        adapter = make_adapter(GridNeRF)
        from landmarksystem_b200.components.data.datasets.ray_utils import get_ray_directions_blender, get_rays_with_directions
        dirs = get_ray_directions_blender(H, W, 60.0).to(dev)
        o, d = get_rays_with_directions(dirs, pose.to(dev))
        d = d / d.norm(dim=-1, keepdim=True)
        with torch.no_grad():
            rgb, _ = ref(torch.cat((o, d, torch.zeros(o.shape[0], 1, device=dev)), -1), N_samples=-1)
        want = (rgb.clamp(0, 1).reshape(H, W, 3) * 255).to(torch.uint8)
        diff = (image[..., :3].int() - want.int()).abs()
        assert image.shape == (H, W, 4) and int(diff.max()) <= 1, int(diff.max())
        assert int(want.float().std()) > 0
        print("ENGINE_BLOCK_MP_RESULTS " + json.dumps({"max_abs_diff_u8": int(diff.max()), "image": [H, W]}), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

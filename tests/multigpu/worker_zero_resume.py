"""Worker (2 GPUs): data-parallel GridNeRF training with the peer-memory ZeRO Adam (every rank holds 1/world of the
Adam moments), stopped after four steps, saved, and resumed in a new trainer.  Each rank must read back ITS OWN shard of
the optimiser state: the resumed run has to land on the parameters of the uninterrupted run, and a shard offered to the
wrong rank has to be refused."""
import json
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from landmarksystem_b200.configs import BaseConfig  # noqa: E402
from landmarksystem_b200.models.gridnerf.gridnerf_trainer import GridNeRFTrainer  # noqa: E402


def batches(rank, n=8, rays=512):
    g = torch.Generator().manual_seed(40 + rank)
    out = []
    for _ in range(n):
        o = torch.tensor([[3.0, 0.0, 0.0]]).expand(rays, 3)
        d = torch.nn.functional.normalize(torch.tensor([[-1.0, 0.0, 0.0]]) + 0.25 * torch.randn(rays, 3, generator=g), dim=-1)
        out.append((torch.cat((o, d), -1).cuda(), torch.rand(rays, 3, generator=g).cuda(), torch.zeros(rays).cuda()))
    return out


def make(root, ckpt=None, **extra):
    conf = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "landmarksystem_b200", "models", "gridnerf",
                        "confs", "synthetic_tiny.py")
    over = {"basedir": root, "device": "cuda", "n_iters": "100", "batch_size": "1024", "DDP": "true", "nSamples": "32",
            "datadir": "ring:3:16x16:20:3", "progress_refresh_rate": "1000", "N_voxel_init": str(32 ** 3),
            "N_voxel_final": str(32 ** 3), "grid_dtype": "bf16"}
    over.update(extra)
    cfg = BaseConfig.from_file(conf, over)
    if ckpt is not None:
        cfg.ckpt = ckpt              # no console form: the field's default is None, so the parser cannot infer its type
    tr = GridNeRFTrainer(cfg)
    tr.model.train()
    return tr


def flat(tr):
    for enc in (tr.module.density_encoding, tr.module.rgb_encoding):
        enc.flush_lazy()
    return torch.cat([p.detach().reshape(-1).float() for p in tr.module.parameters()])


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    root = os.path.join(tempfile.gettempdir(), "lmb_zero_resume")
    data = batches(rank)
    tr = make(root)
    assert getattr(tr.optimizer, "partitioned", False), type(tr.optimizer).__name__
    for it in range(4):
        tr.iteration = it
        torch.manual_seed(1000 + it)            # the stratified sampling jitter of a step depends on the step alone
        tr.train_step(*data[it])
    tr.save_ckpt()
    dist.barrier()
    assert os.path.exists(tr._optim_path()) and f"-sub{rank}" in tr._optim_path()
    for it in range(4, 7):
        tr.iteration = it
        torch.manual_seed(1000 + it)
        tr.train_step(*data[it])
    want = flat(tr)
    # a shard of the other rank must be refused
    other = tr._optim_path().replace(f"-sub{rank}", f"-sub{1 - rank}")
    try:
        tr.optimizer.load_state_dict(torch.load(other, map_location="cuda", weights_only=False)["optimizer"])
        refused = False
    except ValueError:
        refused = True
    assert refused
    tr.optimizer.close()
    del tr
    torch.cuda.empty_cache()
    dist.barrier()
    resumed = make(root, ckpt="auto", start_iters="4")
    for it in range(4, 7):
        resumed.iteration = it
        torch.manual_seed(1000 + it)
        resumed.train_step(*data[it])
    got = flat(resumed)
    err = float((got - want).abs().max())
    scale = float(want.abs().max())
    assert err <= 2e-4 * max(scale, 1.0), (err, scale)
    errs = [None] * world
    dist.all_gather_object(errs, err)
    if rank == 0:
        print("ZERO_RESUME_RESULTS " + json.dumps({"world": world, "max_abs_err": errs}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Worker (2 GPUs): channel-parallel colour head whose all-gather is fused into the tcgen05 MLP's TMA
loads, checked against the unsplit computation."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from landmarksystem_b200.models.gridnerf.gridnerf import RGBDecoder  # noqa: E402
from landmarksystem_b200.ops import fused_mlp  # noqa: E402
from landmarksystem_b200.parallel.channel_gather_mlp import ChannelGatherColourHead  # noqa: E402


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    torch.manual_seed(0)
    L, C = 3, 48
    dec = RGBDecoder([C], [1, 2, 4], 27, view_pe=2, fea_pe=2, featureC=128).cuda()
    for p in dec.parameters():
        dist.broadcast(p.data, src=0)
    N = 1_000_000
    g = torch.Generator(device="cuda").manual_seed(5)
    full = (torch.randn(N, L, C, device="cuda", generator=g) * 0.3).to(torch.bfloat16)      # [level][channel]
    dirs = torch.nn.functional.normalize(torch.randn(N, 3, device="cuda", generator=g), dim=-1)
    cl = C // world
    mine = full[:, :, rank * cl:(rank + 1) * cl].reshape(N, L * cl).contiguous()
    head = ChannelGatherColourHead(dec, L, cl, N)
    out = head(mine, dirs)
    head.packed.check_status()
    head.barrier.check()
    with torch.no_grad():
        ref = fused_mlp.rgb_decoder_forward(dec, dirs, full.reshape(N, L * C).float())
    err = (out - ref).abs().max().item()
    assert err < 2e-2, err

    def run():
        head(mine, dirs)

    for _ in range(3):
        run()
    dist.barrier(); torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        run()
    e.record(); torch.cuda.synchronize()
    ms = torch.tensor([s.elapsed_time(e) / 10], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)

    def baseline():
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        feats = torch.stack([p.view(N, L, cl) for p in parts], 2).reshape(N, L * C)
        with torch.no_grad():
            return fused_mlp.rgb_decoder_forward(dec, dirs, feats.float())

    for _ in range(2):
        baseline()
    torch.cuda.synchronize()
    s.record()
    for _ in range(5):
        baseline()
    e.record(); torch.cuda.synchronize()
    ms_b = torch.tensor([s.elapsed_time(e) / 5], device="cuda")
    dist.all_reduce(ms_b, op=dist.ReduceOp.MAX)
    if rank == 0:
        nvlink = (world - 1) * N * L * cl * 2
        flops = 2.0 * N * (144 * 32 + 160 * 128 + 128 * 128 + 128 * 16)
        print("CHANNEL_GATHER_RESULTS " + json.dumps({"world": world, "rows": N, "max_err": err, "fused_ms": float(ms),
              "nccl_then_mlp_ms": float(ms_b), "nvlink_GBps_per_rank": nvlink / float(ms) / 1e6,
              "tflops": flops / float(ms) / 1e9}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
